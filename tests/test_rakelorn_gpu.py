"""Rakelorn on the GPU against the plain NumPy statement of the design (oracle/ref_rakelorn.py): every mechanism
alone, whole prompts against token-by-token decoding and against portions down to two tokens, batches against
single sequences, reused slots, far keys, looped blocks, router corner cases, odd sizes, and greedy generation
through the library's own loop and scheduler.  Small random models; fp32 mode is held to 1e-4 of the logit
scale, bf16 to 6e-2 (see `close`)."""
import json

import numpy as np
import pytest

from oracle.ref_rakelorn import OracleRakelorn, layer_runs, random_model

pytestmark = pytest.mark.gpu

FP32_BAR, BF16_BAR = 1e-4, 6e-2


def moe(experts=6, top=2, ff=24, identity=1, groups=(1, 1), scale=1.5):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "top": top, "identity": identity, "scale": scale,
                       "groups": {"count": groups[0], "keep": groups[1]}}}


def latent(heads=4, dim=16, rot_dim=8, vdim=24, q_rank=40, kv_rank=48, scale=0.2, base=10000.0, dims=None, mlp=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                      "scale": scale, "rot": {"base": base, "dims": rot_dim if dims is None else dims}},
            "mlp": mlp}


def gru(width=72, mlp=None):
    return {"type": "mingru", "mixer": {"width": width}, "mlp": mlp}


def config(layers, width=64, vocab=97, loop=None, eps=1e-5, embed=3.0):
    c = {"architecture": "Rakelorn", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width,
         "embedding": {"scale": embed}}
    if loop:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


def build(cfg, seed=0, dtype="float32", max_seq_len=128, max_batch_size=1, tensors=None):
    from llama3_np_b200.rakelorn import Rakelorn
    t = random_model(cfg, seed) if tensors is None else tensors
    return Rakelorn(cfg, t, dtype=dtype, max_seq_len=max_seq_len, max_batch_size=max_batch_size), OracleRakelorn(cfg, t)


def err(got, want):
    """largest row error: rms of the mean-free difference over the rms of the mean-free logits"""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return float(np.max(np.sqrt((d * d).mean(-1)) / np.sqrt((w * w).mean())))


def row_errs(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return np.sqrt((d * d).mean(-1)) / np.sqrt((w * w).mean())


def close(got, want, dtype):
    """fp32: every row within the bar.  bf16: a router's choice between two nearly equal scores may fall the other
    way for a token once its inputs are rounded, and that token's row then differs by far more than rounding; so
    nine rows in ten are held to the bar and the typical row to a third of it."""
    e = row_errs(got, want)
    if dtype == "float32":
        return bool(e.max() < FP32_BAR)
    return bool(np.quantile(e, 0.9) < BF16_BAR and np.median(e) < BF16_BAR / 3)


def toks(n, vocab, seed=1):
    return np.random.default_rng(seed).integers(0, vocab, n)


def fresh(o):
    o.reset()
    return o


ALONE = {
    "latent": [latent()],
    "latent_moe": [latent(heads=3, dim=32, rot_dim=16, vdim=8, q_rank=24, kv_rank=80, scale=0.1, mlp=moe())],
    "latent_partial_rotation": [latent(heads=2, dim=8, rot_dim=12, dims=8, base=500.0)],
    "mingru": [gru()],
    "mingru_moe": [gru(width=40, mlp=moe(experts=4, top=1, identity=0))],
    "moe_groups": [gru(width=64, mlp=moe(experts=9, top=3, identity=3, groups=(4, 2), scale=2.0))],
}


@pytest.mark.parametrize("name", sorted(ALONE))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_each_mechanism_alone(name, dtype):
    cfg = config(ALONE[name])
    m, o = build(cfg, seed=3, dtype=dtype)
    ids = toks(40, cfg["vocab"])
    got, resid = m.forward_rows(ids[None], 0, list(range(40)), want_residual=True)
    want, wres = o.run(ids, want_residual=True)
    assert resid.shape == (1, 40, cfg["width"])
    assert close(got, want, dtype)
    if dtype == "float32":
        assert np.allclose(resid, wres, rtol=1e-4, atol=1e-4)
    m.close()


def test_token_shift_reads_the_previous_token_and_zeros_at_the_start():
    """With shift = 1 everywhere the mixer sees only the previous token's input: the first token's mixer input is zero,
    and a portion's first token must fetch the state its predecessor left."""
    cfg = config([gru(width=48), latent(heads=2)], width=32, vocab=40)
    t = random_model(cfg, 4)
    for i in range(2):
        t[f"l{i}.shift"] = np.ones(32)
    m, o = build(cfg, tensors=t)
    ids = toks(12, 40, seed=5)
    want = o.run(ids)
    assert err(m.forward_rows(ids[None], 0, list(range(12))), want) < FP32_BAR
    cut = np.concatenate([m.forward_rows(ids[None, :1], 0, [0]), m.forward_rows(ids[None, 1:3], 1, [0, 1]),
                          m.forward_rows(ids[None, 3:12], 3, list(range(9)))])
    assert err(cut, want) < FP32_BAR
    m.close()


MIXED = [latent(mlp=moe()), gru(mlp=moe(experts=5, top=2, identity=2, groups=(1, 1))), latent(heads=2, dim=8, rot_dim=16, vdim=16, q_rank=16, kv_rank=32, scale=0.3),
         gru(width=96, mlp=moe(experts=8, top=3, identity=0, groups=(2, 1)))]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_then_token_by_token_and_portions(dtype):
    cfg = config(MIXED, loop=(1, 3, 2))
    m, o = build(cfg, seed=5, dtype=dtype, max_seq_len=160)
    n = 150
    ids = toks(n, cfg["vocab"], seed=6)
    want = o.run(ids)
    whole = m.forward_rows(ids[None], 0, list(range(n)))
    assert close(whole, want, dtype)
    # every token alone, from the first one
    one = np.stack([m.forward(ids[None, t:t + 1], t)[0] for t in range(n)])
    assert close(one, want, dtype)
    # portions of changing size, down to two tokens and one; 9 and 8 sit on the border between the few-row and
    # many-row paths of the projections and of the experts
    for sizes in ([37, 3, 2, 2], [2], [64, 1, 5, 2, 31], [9, 8]):
        pos, i, rows = 0, 0, []
        while pos < n:
            c = min(sizes[i % len(sizes)], n - pos)
            i += 1
            rows.append(m.forward_rows(ids[None, pos:pos + c], pos, list(range(c))))
            pos += c
        got = np.concatenate(rows)
        assert close(got, want, dtype)
        if dtype == "float32":
            assert err(got, whole) < 2e-5
    m.close()


def test_looped_block_keeps_one_state_per_pass():
    """A block that runs three times: residuals after every layer run, in a prompt and across a cut, and the caches
    of two passes of the same layer differ."""
    cfg = config([gru(width=40), latent(heads=2, mlp=moe()), gru(width=56)], width=48, vocab=60, loop=(0, 2, 3))
    assert [r[0] for r in layer_runs(cfg)] == [0, 1, 0, 1, 0, 1, 2]
    m, o = build(cfg, seed=7)
    assert m.n_runs == 7
    ids = toks(21, 60, seed=8)
    want, wres = o.run(ids, want_residual=True)
    got, res = m.forward_rows(ids[None, :13], 0, list(range(13)), want_residual=True)
    got2, res2 = m.forward_rows(ids[None, 13:], 13, list(range(8)), want_residual=True)
    assert err(np.concatenate([got, got2]), want) < FP32_BAR
    assert np.allclose(np.concatenate([res, res2], axis=1), wres, rtol=1e-4, atol=1e-4)
    for run in (1, 3, 5):  # the latent layer's three caches
        cache, _ = m.read_state(run)
        st = o.state[run]
        assert np.allclose(cache[:21], np.concatenate([np.stack(st["c"]), np.stack(st["kr"])], axis=1), rtol=1e-4, atol=1e-4)
    assert not np.allclose(m.read_state(1)[0][:21], m.read_state(3)[0][:21], atol=1e-3)
    for run in (0, 2, 4, 6):
        S, _ = m.read_state(run)
        assert np.allclose(S.reshape(-1), o.state[run]["S"], rtol=1e-4, atol=1e-5)
    m.close()


@pytest.mark.parametrize("loop", [None, (0, 3, 1), (0, 3, 2), (2, 3, 4), (1, 1, 2)])
def test_loop_bounds(loop):
    cfg = config([latent(heads=2), gru(width=32, mlp=moe(experts=3, top=2, identity=1)), latent(heads=1, vdim=8)], width=32, vocab=50, loop=loop)
    m, o = build(cfg, seed=9)
    ids = toks(14, 50, seed=10)
    want = o.run(ids)
    got = np.concatenate([m.forward_rows(ids[None, :9], 0, list(range(9))), np.stack([m.forward(ids[None, i:i + 1], i)[0] for i in range(9, 14)])])
    assert err(got, want) < FP32_BAR
    m.close()


def test_long_decoding_matches_the_oracle():
    cfg = config([latent(heads=2, dim=8, rot_dim=8, vdim=8, q_rank=16, kv_rank=24, mlp=moe(experts=4, top=2, ff=16)), gru(width=40)], width=40, vocab=50)
    m, o = build(cfg, seed=11, max_seq_len=400)
    ids = toks(380, 50, seed=12)
    want = o.run(ids)
    m.forward_rows(ids[None, :20], 0, [])
    got = np.stack([m.forward(ids[None, t:t + 1], t)[0] for t in range(20, 380)])
    assert err(got, want[20:]) < FP32_BAR
    m.close()


def test_batch_rows_equal_single_sequences_and_slots_are_reused():
    cfg = config(MIXED, loop=(2, 4, 2))
    t = random_model(cfg, 13)
    m, o = build(cfg, tensors=t, max_seq_len=64, max_batch_size=3)
    ids = np.stack([toks(30, cfg["vocab"], seed=s) for s in (14, 15, 16)])
    batch = m.forward_rows(ids[:, :25], 0, list(range(75)))
    step = m.forward(ids[:, 25:26], 25)
    for b in range(3):
        want = fresh(o).run(ids[b, :26])
        assert err(batch[b * 25:(b + 1) * 25], want[:25]) < FP32_BAR
        assert err(step[b], want[25]) < FP32_BAR
    # slot 0 held sequence 0 up to position 26; a new sequence starting there must not see any of it: not its cache
    # rows, not its recurrent state, not its last token's shifted input
    again = m.forward_rows(ids[2:3, :30], 0, list(range(30)))
    assert err(again, fresh(o).run(ids[2])) < FP32_BAR
    with pytest.raises(RuntimeError):
        m.forward(ids[:1, :1], 7)
    m.close()


def _sharp(t, layer, gain):
    t[f"l{layer}.mix.uq"] = t[f"l{layer}.mix.uq"] * gain
    t[f"l{layer}.mix.uk"] = t[f"l{layer}.mix.uk"] * gain


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_far_keys_dominate_attention(dtype):
    """Queries and keys are scaled up until the softmax is nearly one-hot, so single keys anywhere in the past - the
    first tokens, rows on both sides of every tile and split border - carry the output; hundreds of tokens, in a
    prompt and in decoding, where the keys of a sequence are split over CTAs."""
    cfg = config([latent(heads=3, dim=16, rot_dim=8, vdim=16, q_rank=24, kv_rank=40, scale=1.0)], width=32, vocab=50)
    t = random_model(cfg, 17)
    _sharp(t, 0, 3.0)
    m, o = build(cfg, tensors=t, dtype=dtype, max_seq_len=700)
    ids = toks(650, 50, seed=18)
    want = o.run(ids)
    p = np.stack(o.state[0]["p"])  # the last token's weights: peaked, and not on its neighbours
    assert p.max(axis=1).min() > 0.3 and (649 - p.argmax(axis=1)).max() > 100
    got = m.forward_rows(ids[None, :600], 0, list(range(600)))
    assert close(got, want[:600], dtype)
    tail = np.stack([m.forward(ids[None, i:i + 1], i)[0] for i in range(600, 650)])
    assert close(tail, want[600:], dtype)
    m.close()


def planted_model(seed, token=7, gain=40.0):
    """One layer whose attention every query spends on the rows of ONE token id, wherever they are.  All embeddings
    share a direction u, so a one-dimensional query latent has the same sign for every token and the un-rotated
    (rot.dims = 0) extra query entry is one positive constant; the extra key entry is the embedding's component
    along the planted token's own direction, large for that token only."""
    cfg = config([latent(heads=2, dim=8, rot_dim=2, dims=0, vdim=8, q_rank=1, kv_rank=16, scale=1.0)], width=24, vocab=30, embed=1.0)
    rng = np.random.default_rng(seed)
    t = random_model(cfg, seed, bf16_round=False)
    u = np.zeros(24); u[0] = 1.0
    noise = rng.standard_normal((30, 24)) * 0.5
    noise[:, 0] = 0.0
    t["embed"] = u[None, :] + noise
    t["l0.shift"] = np.zeros(24)
    d = noise[token] / np.linalg.norm(noise[token])
    t["l0.mix.dq"] = 5.0 * u[None, :]
    t["l0.mix.dq.norm"] = np.ones(1)
    uq = t["l0.mix.uq"].reshape(2, 10, 1)
    uq[:, :8, :] *= 0.1
    uq[:, 8, 0] = 1.0
    uq[:, 9, 0] = 0.0
    t["l0.mix.uq"] = uq.reshape(20, 1)
    dkv = t["l0.mix.dkv"]
    dkv[16] = gain * d
    dkv[17] = 0.0
    for k in t:  # onto the bf16 grid
        a = np.ascontiguousarray(t[k], dtype=np.float32)
        t[k] = ((a.view(np.uint32) + 0x8000) & 0xFFFF0000).astype(np.uint32).view(np.float32).reshape(a.shape).astype(np.float64)
    return cfg, t


@pytest.mark.parametrize("planted", [0, 31, 32, 257])
def test_one_planted_key_is_found_from_everywhere(planted):
    """The planted token sits once in the sequence: at the first position, at a tile's last row, at the next tile's
    first row, far inside.  Every later token must put its weight there, in a prompt and token by token."""
    cfg, t = planted_model(19)
    m, o = build(cfg, tensors=t, max_seq_len=420)
    ids = toks(400, 30, seed=20 + planted)
    ids[ids == 7] = 8
    ids[planted] = 7
    want = o.run(ids)
    p = np.stack(o.state[0]["p"])
    assert p[:, planted].min() > 0.9, p[:, planted]
    got = np.concatenate([m.forward_rows(ids[None, :300], 0, list(range(300))),
                          np.stack([m.forward(ids[None, i:i + 1], i)[0] for i in range(300, 400)])])
    assert err(got, want) < FP32_BAR
    # and without the planted row the answer is another one: the row matters
    ids2 = ids.copy()
    ids2[planted] = 9
    assert err(fresh(o).run(ids2)[-1:], want[-1:]) > 10 * FP32_BAR
    m.close()


def test_router_negative_choices_and_group_limits():
    """All corrections strongly negative: every choice score is below zero, so a slot masked by its group must count as
    minus infinity (a zero would win).  Also top = all slots of the kept groups, and identity slots in a kept group."""
    for groups, top, experts, identity in (((3, 1), 3, 7, 2), ((2, 1), 2, 3, 1), ((4, 3), 5, 8, 0), ((1, 1), 4, 2, 2)):
        cfg = config([gru(width=32, mlp=moe(experts=experts, top=top, identity=identity, groups=groups, ff=16, scale=0.7))], width=32, vocab=40)
        t = random_model(cfg, 21)
        t["l0.mlp.correction"] = t["l0.mlp.correction"] - 1.0
        t["l0.mlp.correction"] = np.asarray(t["l0.mlp.correction"], np.float32).astype(np.float64)
        m, o = build(cfg, tensors=t)
        ids = toks(30, 40, seed=22)
        want = o.run(ids)
        got = np.concatenate([m.forward_rows(ids[None, :24], 0, list(range(24))), m.forward_rows(ids[None, 24:], 24, list(range(6)))])
        assert err(got, want) < FP32_BAR, (groups, top)
        m.close()


ODD = {
    # sizes the vector paths do not take, and values the usual configs make equal or 1
    "width_not_8": config([latent(heads=3, dim=12, rot_dim=6, vdim=10, q_rank=20, kv_rank=28, mlp=moe(experts=3, top=1, ff=10, identity=0)), gru(width=36)], width=44, vocab=33),
    "width_not_4": config([gru(width=25, mlp=moe(experts=2, top=2, ff=7, identity=1)), latent(heads=1, dim=5, rot_dim=2, vdim=3, q_rank=7, kv_rank=9, scale=1.0)], width=30, vocab=40, eps=1e-3, embed=1.0),
    "row_not_4": config([latent(heads=5, dim=6, rot_dim=6, vdim=6, q_rank=10, kv_rank=13, scale=0.5)], width=40, vocab=25),
    "many_heads": config([latent(heads=35, dim=4, rot_dim=4, vdim=2, q_rank=12, kv_rank=8, scale=0.5)], width=24, vocab=25),
    "wide_values": config([latent(heads=2, dim=8, rot_dim=8, vdim=72, q_rank=12, kv_rank=136, scale=0.3, mlp=moe(experts=2, top=1, ff=80, identity=0))], width=48, vocab=31),
    "long_latent": config([latent(heads=2, dim=8, rot_dim=16, vdim=8, q_rank=8, kv_rank=600, scale=0.3)], width=32, vocab=31),
    "no_feed_forward": config([gru(width=16), latent(heads=2), gru(width=128)], width=16, vocab=20, loop=(1, 2, 2)),
}


@pytest.mark.parametrize("name", sorted(ODD))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_odd_sizes(name, dtype):
    cfg = ODD[name]
    m, o = build(cfg, seed=23, dtype=dtype)
    ids = toks(33, cfg["vocab"], seed=24)
    want = o.run(ids)
    got = np.concatenate([m.forward_rows(ids[None, :20], 0, list(range(20))), m.forward_rows(ids[None, 20:22], 20, [0, 1]),
                          np.stack([m.forward(ids[None, i:i + 1], i)[0] for i in range(22, 33)])])
    assert close(got, want, dtype)
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_library_loop(dtype):
    cfg = config(MIXED, loop=(0, 2, 2))
    m, o = build(cfg, seed=25, dtype=dtype, max_seq_len=96, max_batch_size=2)
    prompts = np.stack([toks(12, cfg["vocab"], seed=s) for s in (26, 27)])
    lazy = np.concatenate(list(m.generate(prompts, 40)), axis=1)
    bulk = m.generate_all(prompts, 40)
    assert np.array_equal(lazy, bulk)
    # teacher-forced check: every emitted token is the oracle's argmax for the same prefix, unless the oracle's
    # top two are closer than the mode's error bar
    margin = 1e-3 if dtype == "float32" else 0.2
    for b in range(2):
        seq = np.concatenate([prompts[b], bulk[b]])
        lg = fresh(o).run(seq[:-1])
        for i in range(40):
            row = lg[11 + i]
            top = np.sort(row)[-2:]
            if top[1] - top[0] > margin * np.std(row):
                assert int(np.argmax(row)) == int(bulk[b, i]), f"sequence {b}, new token {i}"
    m.close()


def test_scheduler_runs_unequal_prompts_as_each_alone():
    cfg = config(MIXED[:3], loop=(1, 2, 2))
    m, _ = build(cfg, seed=28, max_seq_len=64, max_batch_size=2)
    prompts = [toks(n, cfg["vocab"], seed=29 + n) for n in (5, 9, 5, 2, 9)]
    outs = m.generate_ragged(prompts, 10)
    for p, got in zip(prompts, outs):
        assert np.array_equal(got, m.generate_all(p[None], 10)[0])
    m.close()


def _write_folder(tmp_path, cfg, t):
    from test_risalix_cpu import write_safetensors
    write_safetensors(tmp_path / "model.safetensors", t)
    (tmp_path / "config.json").write_text(json.dumps(cfg))


def test_registry_and_checkpoint_folder(tmp_path):
    from llama3_np_b200.models import load_model
    cfg = config([latent(heads=2, mlp=moe()), gru(width=24)], width=32, vocab=41, loop=(0, 1, 2))
    t = random_model(cfg, 30)
    _write_folder(tmp_path, cfg, t)
    m = load_model(str(tmp_path), dtype="float32", max_seq_len=32)
    assert type(m).__name__ == "Rakelorn"
    ids = toks(16, 41, seed=31)
    assert err(m.forward_rows(ids[None], 0, list(range(16))), OracleRakelorn(cfg, t).run(ids)) < FP32_BAR
    m.close()


def test_trace_runner_replays_a_trace(tmp_path):
    """bin/trace_run as a user runs it: two requests after one another through the same slot, portions cut in odd
    places and longer than one forward call."""
    import os
    import subprocess
    import sys
    from conftest import ROOT
    cfg = config([latent(heads=2, mlp=moe()), gru(width=24, mlp=moe(experts=3, top=2, identity=0))], width=32, vocab=41, loop=(0, 2, 2))
    t = random_model(cfg, 32)
    _write_folder(tmp_path, cfg, t)
    o = OracleRakelorn(cfg, t)
    reqs = {"a": toks(23, 41, seed=33), "b": toks(9, 41, seed=34)}
    want = {k: fresh(o).run(v) for k, v in reqs.items()}
    steps, expect, n = [], {}, 0
    for rid, cuts in (("a", [11, 1, 2, 9]), ("b", [9])):
        pos = 0
        for c in cuts:
            w = [0, c - 1] if c > 1 else [0]
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [int(x) for x in reqs[rid][pos:pos + c]], "want": w}],
                          "end": [rid] if pos + c == len(reqs[rid]) else []})
            expect[n] = want[rid][[pos + i for i in w]]
            pos += c
            n += 1
    steps.append({"step": n, "entries": [], "end": []})
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(tmp_path), "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "64", "--piece", "5"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(n + 1)]
    for i, e in expect.items():
        got = np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, 41)
        assert err(got, e) < FP32_BAR, i


def test_generate_command_prints_the_loop_s_tokens(tmp_path):
    import os
    import subprocess
    import sys
    from conftest import ROOT
    from llama3_np_b200.models import load_model
    cfg = config([gru(width=24), latent(heads=2, mlp=moe())], width=32, vocab=47)
    _write_folder(tmp_path, cfg, random_model(cfg, 35))
    prompts = np.stack([toks(7, 47, seed=s) for s in (36, 37)])
    (tmp_path / "prompts.txt").write_text("\n".join(" ".join(str(int(x)) for x in p) for p in prompts) + "\n")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "generate"), "--model", str(tmp_path), "--dtype", "float32",
                        "--batch-file", str(tmp_path / "prompts.txt"), "--new", "12"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    printed = np.array([[int(x) for x in line.split()] for line in r.stdout.strip().splitlines()[-2:]])
    m = load_model(str(tmp_path), dtype="float32", max_seq_len=19, max_batch_size=2)
    assert np.array_equal(printed, m.generate_all(prompts, 12))
    m.close()


def test_larger_shapes_take_the_tensor_core_projections():
    """Width 256 and 70 rows: in bf16 mode the projections of a portion run as tcgen05 GEMMs, the experts as one
    masked GEMM over all of them; decode rows read only the chosen experts."""
    cfg = config([latent(heads=4, dim=32, rot_dim=32, vdim=64, q_rank=128, kv_rank=128, scale=0.1, mlp=moe(experts=8, top=2, ff=64, identity=1, groups=(3, 2))),
                  gru(width=256, mlp=moe(experts=4, top=2, ff=128, identity=0))], width=256, vocab=300, loop=(0, 2, 2))
    for dtype in ("bfloat16", "float32"):
        m, o = build(cfg, seed=38, dtype=dtype, max_seq_len=128)
        ids = toks(80, 300, seed=39)
        want = o.run(ids)
        got = np.concatenate([m.forward_rows(ids[None, :70], 0, list(range(70))),
                              np.stack([m.forward(ids[None, i:i + 1], i)[0] for i in range(70, 80)])])
        assert close(got, want, dtype)
        m.close()
