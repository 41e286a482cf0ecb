"""Plain NumPy (float64) statement of the Rakelorn decoder, one function per mechanism.

The oracle of `llama3_np_b200.rakelorn`: it shares no code with the product path, runs token by
token, and keeps every intermediate in float64.  Nothing here is fast.

Notation: `x` is the residual row (width W), `h` a sublayer's input row, `P` a dict of one layer's
tensors with the `l<i>.` prefix removed, `st` the mutable per-sequence state of one layer RUN (a
layer inside the loop runs several times per token and owns one state per pass).

    x_0 = s_e * E[token]
    pass t of the looped block:  x += T[t]   (once, ahead of the block's first layer)
    layer:  h = n1 * x / rms(x);  h~ = h + (h_prev - h) * shift;  x += mixer(h~)
            x += moe(n2 * x / rms(x))
    logits = head (n_f * x / rms(x))
with n1, n2, n_f single numbers and h_prev the previous token's un-shifted h (zeros at position 0).
"""
from __future__ import annotations

import numpy as np


# ------------------------------------------------------------------ scalar functions
def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softmax(z):
    e = np.exp(z - np.max(z))
    return e / e.sum()


def rotate_pairs(v, pos, dims, base):
    """Rotary position on the first `dims` entries of v, entry 2i paired with 2i + 1; the angle of
    pair i at position pos is pos * base^(-2i / dims).  The remaining entries pass unchanged."""
    out = np.array(v, dtype=np.float64)
    i = np.arange(dims // 2)
    ang = pos * np.power(float(base), -2.0 * i / dims)
    c, s = np.cos(ang), np.sin(ang)
    a, b = out[0:dims:2].copy(), out[1:dims:2].copy()
    out[0:dims:2] = a * c - b * s
    out[1:dims:2] = b * c + a * s
    return out


# ------------------------------------------------------------------ token shift
def token_shift(h, mu, st):
    """h + (previous h - h) * mu, the previous h taken before ITS shift; zeros ahead of the first token."""
    prev = st.get("h_prev")
    if prev is None:
        prev = np.zeros_like(h)
    st["h_prev"] = h.copy()
    return h + (prev - h) * mu


# ------------------------------------------------------------------ mixers (one token each)
def latent_attention_step(h, pos, P, mc, eps, st):
    """Attention whose keys and values are expanded from one cached latent row per token.

    q-side: cq = w_dq_norm * unit(Wdq h); per head q = [q_c (dim) | q_r (rot_dim)] = rows of Wuq cq.
    kv-side: Wdkv h = [c_raw (kv_rank) | k_r (rot_dim)]; c = w_dkv_norm * unit(c_raw) and the rotated k_r are
    the cache.  Head j: score(i) = scale * (q_c . (Wuk_j c_i) + rot(q_r) . rot(k_r,i)), softmax over i <= pos,
    o_j = sigmoid(Wg h)_j * sum_i p_i Wuv_j c_i;  y = Wo concat(o)."""
    H, dn, dr, dv, rank = mc["heads"], mc["dim"], mc["rot_dim"], mc["vdim"], mc["kv_rank"]
    rot = mc["rot"]
    cq = rms_unit(P["mix.dq"] @ h, eps) * P["mix.dq.norm"]
    q = (P["mix.uq"] @ cq).reshape(H, dn + dr)
    kv = P["mix.dkv"] @ h
    c = rms_unit(kv[:rank], eps) * P["mix.dkv.norm"]
    kr = rotate_pairs(kv[rank:], pos, rot["dims"], rot["base"])
    st.setdefault("c", []).append(c)
    st.setdefault("kr", []).append(kr)
    C = np.stack(st["c"])          # [T, rank]
    KR = np.stack(st["kr"])        # [T, dr]
    gate = sigmoid(P["mix.g"] @ h)
    Wuk = P["mix.uk"].reshape(H, dn, rank)
    Wuv = P["mix.uv"].reshape(H, dv, rank)
    out = np.zeros((H, dv))
    st["p"] = []                   # the last token's attention weights, head by head (tests look at them)
    for j in range(H):
        qr = rotate_pairs(q[j, dn:], pos, rot["dims"], rot["base"])
        K = C @ Wuk[j].T           # [T, dn]
        V = C @ Wuv[j].T           # [T, dv]
        p = softmax((K @ q[j, :dn] + KR @ qr) * mc["scale"])
        st["p"].append(p)
        out[j] = gate[j] * (p @ V)
    return P["mix.o"] @ out.reshape(-1)


def mingru_step(h, P, mc, st):
    """z = sigmoid(Wz h + bz), u = Wx h + bx, cand = u + 1/2 (u >= 0) | sigmoid(u) (u < 0),
    S <- (1 - z) S + z cand (element by element, S = 0 ahead of the first token), y = Wo (S * silu(Wg h))."""
    z = sigmoid(P["mix.z"] @ h + P["mix.z.b"])
    u = P["mix.x"] @ h + P["mix.x.b"]
    cand = np.where(u >= 0, u + 0.5, sigmoid(u))
    S = st.get("S")
    if S is None:
        S = np.zeros(mc["width"])
    S = (1.0 - z) * S + z * cand
    st["S"] = S
    return P["mix.o"] @ (S * silu(P["mix.g"] @ h))


# ------------------------------------------------------------------ feed-forward
def route(h, P, rc):
    """(chosen slots, their weights).  s = softmax(Wr h) over experts and identity slots; choice = s + correction;
    slots outside the `keep` best groups (a group's rank is its largest choice) are out; the `top` largest
    choices win; weight = s * scale, not renormalised."""
    s = softmax(P["mlp.router"] @ h)
    choice = s + P["mlp.correction"]
    n = len(s)
    g = rc.get("groups") or {"count": 1, "keep": 1}
    per = n // g["count"]
    best = choice.reshape(g["count"], per).max(axis=1)
    kept = np.argsort(-best, kind="stable")[: g["keep"]]
    masked = np.full(n, -np.inf)
    for gi in kept:
        masked[gi * per:(gi + 1) * per] = choice[gi * per:(gi + 1) * per]
    chosen = np.argsort(-masked, kind="stable")[: rc["top"]]
    return chosen, s[chosen] * rc["scale"]


def moe(h, P, mlp):
    """sum over the chosen slots of weight * (Wdown relu(Wup h)^2), an identity slot giving weight * h."""
    rc = mlp["router"]
    chosen, w = route(h, P, rc)
    y = np.zeros_like(h)
    for e, we in zip(chosen, w):
        if e >= rc["experts"]:
            y += we * h
        else:
            a = np.maximum(P[f"mlp.e{e}.up"] @ h, 0.0) ** 2
            y += we * (P[f"mlp.e{e}.down"] @ a)
    return y


# ------------------------------------------------------------------ the model
def layer_runs(config):
    """[(layer index, pass number or None, first of its pass)] in the order the layers run."""
    n = len(config["layers"])
    lp = config.get("loop")
    if not lp:
        return [(i, None, False) for i in range(n)]
    runs = [(i, None, False) for i in range(lp["start"])]
    for t in range(lp["times"]):
        runs += [(i, t, i == lp["start"]) for i in range(lp["start"], lp["stop"])]
    return runs + [(i, None, False) for i in range(lp["stop"], n)]


class OracleRakelorn:
    def __init__(self, config, tensors):
        self.cfg = config
        self.T = {k: np.asarray(v, dtype=np.float64) for k, v in tensors.items()}
        self.eps = float(config["norm"]["eps"])
        self.runs = layer_runs(config)
        self.per_layer = []
        for i in range(len(config["layers"])):
            pre = f"l{i}."
            self.per_layer.append({k[len(pre):]: v for k, v in self.T.items() if k.startswith(pre)})
        self.reset()

    def reset(self):
        self.state = [dict() for _ in self.runs]
        self.pos = 0

    def step(self, token, want_residual=False):
        """One token -> logits (and the residual row after every layer run)."""
        cfg, T = self.cfg, self.T
        x = T["embed"][int(token)] * float(cfg["embedding"]["scale"])
        trace = []
        for (li, t, first), st in zip(self.runs, self.state):
            if first:
                x = x + T["loop.step"][t]
            lc, P = cfg["layers"][li], self.per_layer[li]
            h = token_shift(rms_unit(x, self.eps) * P["norm1"], P["shift"], st)
            if lc["type"] == "latent_attention":
                x = x + latent_attention_step(h, self.pos, P, lc["mixer"], self.eps, st)
            elif lc["type"] == "mingru":
                x = x + mingru_step(h, P, lc["mixer"], st)
            else:
                raise ValueError(lc["type"])
            if lc.get("mlp") is not None:
                x = x + moe(rms_unit(x, self.eps) * P["norm2"], P, lc["mlp"])
            trace.append(x.copy())
        self.pos += 1
        logits = T["head"] @ (rms_unit(x, self.eps) * T["final.norm"])
        return (logits, np.stack(trace)) if want_residual else logits

    def run(self, tokens, want_residual=False):
        """Continue the sequence with `tokens`; logits [n, vocab] (and residuals [runs, n, W])."""
        outs = [self.step(t, want_residual) for t in tokens]
        if want_residual:
            return np.stack([o[0] for o in outs]), np.stack([o[1] for o in outs], axis=1)
        return np.stack(outs)


def random_model(config, seed, bf16_round=True):
    """Random tensors for a configuration (names and shapes as a checkpoint has them)."""
    rng = np.random.default_rng(seed)
    W, V = config["width"], config["vocab"]

    def mat(o, i, gain=1.0):
        return rng.standard_normal((o, i)) * gain / np.sqrt(i)

    t = {"embed": rng.standard_normal((V, W)) * 0.1, "head": mat(V, W), "final.norm": np.asarray(1.0 + 0.1 * rng.standard_normal())}
    lp = config.get("loop")
    if lp:
        t["loop.step"] = rng.standard_normal((lp["times"], W)) * 0.3
    for i, lc in enumerate(config["layers"]):
        p, mc = f"l{i}.", lc["mixer"]
        t[p + "norm1"] = np.asarray(1.0 + 0.1 * rng.standard_normal())
        t[p + "shift"] = rng.uniform(0.0, 1.0, W)
        if lc["type"] == "latent_attention":
            H, dn, dr, dv = mc["heads"], mc["dim"], mc["rot_dim"], mc["vdim"]
            t[p + "mix.dq"] = mat(mc["q_rank"], W)
            t[p + "mix.dq.norm"] = 1.0 + 0.1 * rng.standard_normal(mc["q_rank"])
            t[p + "mix.uq"] = mat(H * (dn + dr), mc["q_rank"], 2.0)
            t[p + "mix.dkv"] = mat(mc["kv_rank"] + dr, W, 2.0)
            t[p + "mix.dkv.norm"] = 1.0 + 0.1 * rng.standard_normal(mc["kv_rank"])
            t[p + "mix.uk"] = mat(H * dn, mc["kv_rank"], 2.0)
            t[p + "mix.uv"] = mat(H * dv, mc["kv_rank"])
            t[p + "mix.g"] = mat(H, W)
            t[p + "mix.o"] = mat(W, H * dv)
        else:
            n = mc["width"]
            t[p + "mix.z"] = mat(n, W)
            t[p + "mix.z.b"] = rng.standard_normal(n)
            t[p + "mix.x"] = mat(n, W)
            t[p + "mix.x.b"] = 0.5 * rng.standard_normal(n)
            t[p + "mix.g"] = mat(n, W)
            t[p + "mix.o"] = mat(W, n)
        mlp = lc.get("mlp")
        if mlp is not None:
            rc, ff = mlp["router"], mlp["expert"]["ff"]
            t[p + "norm2"] = np.asarray(1.0 + 0.1 * rng.standard_normal())
            for e in range(rc["experts"]):
                t[p + f"mlp.e{e}.up"] = mat(ff, W)
                t[p + f"mlp.e{e}.down"] = mat(W, ff)
            n = rc["experts"] + rc.get("identity", 0)
            t[p + "mlp.router"] = mat(n, W, 3.0)
            t[p + "mlp.correction"] = 0.05 * rng.standard_normal(n)
    if bf16_round:  # values a bfloat16 checkpoint can hold: both precisions of the product then read the same weights
        for k in t:
            a = np.ascontiguousarray(t[k], dtype=np.float32)
            u = a.view(np.uint32)
            u = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
            t[k] = u.view(np.float32).reshape(a.shape).astype(np.float64)
    return t
