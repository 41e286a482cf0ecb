"""Plain NumPy (float64) statement of the Risalix decoder, one function per mechanism.

The oracle of `llama3_np_b200.risalix`: it shares no code with the product path, runs token by
token, and keeps every intermediate in float64.  Nothing here is fast.

Notation: `h` is a mixer's input row (width), `P` a dict of this layer's tensors with the
`l<i>.` prefix removed, `st` the mutable per-sequence state of that layer.

Layer (post-norm residual, `m` = residual_mult, `N` = RMS norm with weight 1 + w):
    x += m * N1(mixer(x));  x += m * N2(ff(x)) when the layer has a feed-forward;
    x += m * rms(y) * side.norm  with  y = side.proj (gelu(side.gate x) * E[token, layer slice]).
"""
from __future__ import annotations

import numpy as np


# ------------------------------------------------------------------ scalar functions
def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


# ------------------------------------------------------------------ mixers (one token each)
def lightning_step(h, P, mc, eps, st):
    """Linear attention with one fixed decay per head: S <- decay S + k v^T, o = S^T q."""
    H, dk, dv = mc["heads"], mc["dim"], mc["vdim"]
    q = silu(P["mix.q"] @ h).reshape(H, dk)
    k = silu(P["mix.k"] @ h).reshape(H, dk)
    v = silu(P["mix.v"] @ h).reshape(H, dv)
    if "S" not in st:
        st["S"] = np.zeros((H, dk, dv))
    lam = np.asarray(mc["decay"], dtype=np.float64).reshape(H, 1, 1)
    st["S"] = lam * st["S"] + k[:, :, None] * v[:, None, :]
    o = np.einsum("hkv,hk->hv", st["S"], q).reshape(-1)
    o = rms_unit(o, eps) * P["mix.norm"]
    o = o * sigmoid(P["mix.g"] @ h)
    return P["mix.o"] @ o


def _short_conv(name, z, P, st):
    """Causal depthwise convolution over time; the last column of the taps multiplies the current input."""
    w = P[name + ".conv"]
    taps = w.shape[1]
    hist = st.setdefault(name + ".hist", np.zeros((taps - 1, z.shape[0])))
    window = np.concatenate([hist, z[None, :]], axis=0)  # oldest first, current last
    st[name + ".hist"] = window[1:] if taps > 1 else hist
    return silu(np.einsum("tc,ct->c", window, w))


def channel_delta_step(h, P, mc, eps, st):
    """Gated delta rule with one decay per head and key channel."""
    H, G, dk, dv = mc["heads"], mc["kv_heads"], mc["dim"], mc["vdim"]
    q = _short_conv("mix.q", P["mix.q"] @ h, P, st).reshape(G, dk)
    k = _short_conv("mix.k", P["mix.k"] @ h, P, st).reshape(G, dk)
    v = _short_conv("mix.v", P["mix.v"] @ h, P, st).reshape(H, dv)
    q = q / np.sqrt(np.sum(q * q, axis=-1, keepdims=True) + 1e-6) * dk ** -0.5
    k = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
    beta = sigmoid(P["mix.b"] @ h)  # [H]
    dt = softplus(P["mix.a2"] @ (P["mix.a1"] @ h) + P["mix.dt_bias"]).reshape(H, dk)
    g = np.exp(-np.exp(P["mix.A_log"]).reshape(H, 1) * dt)  # [H, dk]
    gate = sigmoid(P["mix.g2"] @ (P["mix.g1"] @ h)).reshape(H, dv)
    if "S" not in st:
        st["S"] = np.zeros((H, dk, dv))
    out = np.zeros((H, dv))
    rep = H // G
    for i in range(H):
        S = st["S"][i]
        qi, ki = q[i // rep], k[i // rep]
        S = g[i][:, None] * S
        u = beta[i] * (v[i] - S.T @ ki)
        S = S + np.outer(ki, u)
        st["S"][i] = S
        out[i] = S.T @ qi
    out = rms_unit(out, eps) * P["mix.norm"][None, :] * gate
    return P["mix.o"] @ out.reshape(-1)


def attention_step(h, P, mc, eps, st):
    """Causal softmax attention without positions; the values are the un-normalised keys."""
    H, G, dk = mc["heads"], mc["kv_heads"], mc["dim"]
    q = P["mix.q"] @ h
    k = P["mix.k"] @ h
    vals = k.reshape(G, dk).copy()
    q = (rms_unit(q, eps) * P["mix.q.norm"]).reshape(H, dk)
    k = (rms_unit(k, eps) * P["mix.k.norm"]).reshape(G, dk)
    st.setdefault("K", []).append(k)
    st.setdefault("V", []).append(vals)
    K = np.stack(st["K"])  # [T, G, dk]
    V = np.stack(st["V"])
    gate = sigmoid(P["mix.g"] @ h)  # [H]
    rep = H // G
    out = np.zeros((H, V.shape[-1]))
    for i in range(H):
        s = K[:, i // rep, :] @ q[i] * mc["scale"]
        p = np.exp(s - s.max())
        p /= p.sum()
        out[i] = gate[i] * (p @ V[:, i // rep, :])
    return P["mix.o"] @ out.reshape(-1)


MIXERS = {"lightning": lightning_step, "channel_delta": channel_delta_step, "attention": attention_step}


# ------------------------------------------------------------------ the rest of a layer
def dense_ff(x, P):
    return P["mlp.down"] @ (gelu_tanh(P["mlp.gate"] @ x) * (P["mlp.up"] @ x))


def side_input(x, e, P, eps):
    y = P["side.proj"] @ (gelu_tanh(P["side.gate"] @ x) * e)
    return rms_unit(y, eps) * P["side.norm"]


class OracleRisalix:
    """`step(token)` feeds one token of one sequence and returns its logits; `new_state()` starts a sequence."""

    def __init__(self, config: dict, tensors: dict):
        self.cfg = config
        self.t = {k: np.asarray(v, dtype=np.float64) for k, v in tensors.items()}
        self.eps = float(config["norm"]["eps"])
        self.m = float(config["residual_mult"])
        self.sd = int((config.get("token_side") or {}).get("dim", 0))
        self.layers = []
        for i, lc in enumerate(config["layers"]):
            pre = f"l{i}."
            self.layers.append((lc, {k[len(pre):]: v for k, v in self.t.items() if k.startswith(pre)}))

    def new_state(self):
        return [dict() for _ in self.layers]

    def step(self, token: int, state, trace=None):
        x = self.t["embed"][token].copy()
        for i, (lc, P) in enumerate(self.layers):
            y = MIXERS[lc["type"]](x, P, lc["mixer"], self.eps, state[i])
            x = x + self.m * rms_unit(y, self.eps) * (1.0 + P["norm1"])
            if lc["mlp"] is not None:
                assert lc["mlp"]["kind"] == "dense"
                y = dense_ff(x, P)
                x = x + self.m * rms_unit(y, self.eps) * (1.0 + P["norm2"])
            if self.sd:
                e = self.t["side.embed"][token, i * self.sd:(i + 1) * self.sd]
                x = x + self.m * side_input(x, e, P, self.eps)
            if trace is not None:
                trace.append(x.copy())
        x = rms_unit(x, self.eps) * (1.0 + self.t["final.norm"])
        return self.t["head"] @ x

    def run(self, tokens, state=None):
        """Logits [len(tokens), vocab] of a sequence (continuing `state` when given)."""
        state = self.new_state() if state is None else state
        return np.stack([self.step(int(t), state) for t in tokens])


def random_model(config: dict, seed: int = 0, bf16_grid: bool = True):
    """Random tensors of a config, in the checkpoint's names and shapes.  `bf16_grid` rounds them to values
    that bfloat16 holds exactly, as a checkpoint would."""
    rng = np.random.default_rng(seed)
    W, V, sd = config["width"], config["vocab"], (config.get("token_side") or {}).get("dim", 0)
    n = len(config["layers"])
    t = {}

    def lin(o, i, gain=1.0):
        return rng.standard_normal((o, i)) * gain / np.sqrt(i)

    t["embed"] = rng.standard_normal((V, W))
    if sd:
        t["side.embed"] = rng.standard_normal((V, sd * n))
    for i, lc in enumerate(config["layers"]):
        p, mc = f"l{i}.", lc["mixer"]
        t[p + "norm1"] = 0.1 * rng.standard_normal(W)
        if lc["type"] == "lightning":
            H, dk, dv = mc["heads"], mc["dim"], mc["vdim"]
            t[p + "mix.q"], t[p + "mix.k"] = lin(H * dk, W, 2.0), lin(H * dk, W, 2.0)
            t[p + "mix.v"], t[p + "mix.g"] = lin(H * dv, W, 2.0), lin(H * dv, W)
            t[p + "mix.o"] = lin(W, H * dv)
            t[p + "mix.norm"] = 1.0 + 0.1 * rng.standard_normal(H * dv)
        elif lc["type"] == "channel_delta":
            H, G, dk, dv, taps = mc["heads"], mc["kv_heads"], mc["dim"], mc["vdim"], mc["conv"]
            r = max(2, W // 8)
            for nm, rows in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                t[p + f"mix.{nm}"] = lin(rows, W, 2.0)
                t[p + f"mix.{nm}.conv"] = rng.standard_normal((rows, taps)) / np.sqrt(taps)
            t[p + "mix.b"] = lin(H, W)
            t[p + "mix.A_log"] = np.log(rng.uniform(0.5, 4.0, H))
            t[p + "mix.norm"] = 1.0 + 0.1 * rng.standard_normal(dv)
            t[p + "mix.a1"], t[p + "mix.a2"] = lin(r, W), lin(H * dk, r)
            t[p + "mix.dt_bias"] = rng.uniform(-3.0, 0.0, H * dk)
            t[p + "mix.g1"], t[p + "mix.g2"] = lin(r, W), lin(H * dv, r)
            t[p + "mix.o"] = lin(W, H * dv)
        else:
            H, G, dk = mc["heads"], mc["kv_heads"], mc["dim"]
            t[p + "mix.q"], t[p + "mix.k"] = lin(H * dk, W), lin(G * dk, W)
            t[p + "mix.q.norm"] = 1.0 + 0.1 * rng.standard_normal(H * dk)
            t[p + "mix.k.norm"] = 1.0 + 0.1 * rng.standard_normal(G * dk)
            t[p + "mix.g"] = lin(H, W)
            t[p + "mix.o"] = lin(W, H * dk)
        if lc["mlp"] is not None:
            ff = lc["mlp"]["ff"]
            t[p + "norm2"] = 0.1 * rng.standard_normal(W)
            t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"] = lin(ff, W), lin(ff, W), lin(W, ff)
        if sd:
            t[p + "side.gate"], t[p + "side.proj"] = lin(sd, W), lin(W, sd)
            t[p + "side.norm"] = 1.0 + 0.1 * rng.standard_normal(W)
    t["final.norm"] = 0.1 * rng.standard_normal(W)
    t["head"] = lin(V, W)
    if bf16_grid:
        for k in t:
            a = np.asarray(t[k], dtype=np.float32)
            bits = a.view(np.uint32)
            bits = ((bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)  # round to nearest even
            t[k] = bits.view(np.float32).astype(np.float64)
    return t
