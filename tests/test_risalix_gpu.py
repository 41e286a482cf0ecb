"""Risalix on the GPU against the plain NumPy statement of the design (oracle/ref_risalix.py): every mixer
alone, whole prompts against token-by-token decoding and against portions down to two tokens, batches
against single sequences, reused slots, far keys and long decays, odd sizes, and greedy generation through
the library's own loop.  Small random models; fp32 mode is held to 1e-4 of the logit scale, bf16 to 6e-2."""
import numpy as np
import pytest

from oracle.ref_risalix import OracleRisalix, random_model

pytestmark = pytest.mark.gpu

FP32_BAR, BF16_BAR = 1e-4, 6e-2


def attn(heads=4, kv=2, dim=16, scale=0.3, ff=0):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def lightning(heads=2, dim=16, vdim=16, decay=(0.7, 0.98), ff=0):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def delta(heads=4, kv=2, dim=16, vdim=8, conv=3, ff=0):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(layers, width=64, vocab=97, side=8, mult=0.5, eps=1e-5):
    c = {"architecture": "Risalix", "layers": layers, "norm": {"eps": eps}, "residual_mult": mult, "vocab": vocab,
         "width": width}
    if side:
        c["token_side"] = {"dim": side}
    return c


def build(cfg, seed=0, dtype="float32", max_seq_len=128, max_batch_size=1, tensors=None):
    from llama3_np_b200.risalix import Risalix
    t = random_model(cfg, seed) if tensors is None else tensors
    return Risalix(cfg, t, dtype=dtype, max_seq_len=max_seq_len, max_batch_size=max_batch_size), OracleRisalix(cfg, t)


def err(got, want):
    """largest row error: rms of the mean-free difference over the rms of the mean-free logits"""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return float(np.max(np.sqrt((d * d).mean(-1)) / np.sqrt((w * w).mean())))


def toks(n, vocab, seed=1):
    return np.random.default_rng(seed).integers(0, vocab, n)


ALONE = {
    "attention": [attn(ff=0)],
    "attention_mlp": [attn(heads=6, kv=2, dim=32, scale=0.11, ff=96)],
    "lightning": [lightning()],
    "lightning_wide_v": [lightning(heads=3, dim=16, vdim=32, decay=(0.5, 0.9, 0.999), ff=80)],
    "delta": [delta()],
    "delta_full_heads": [delta(heads=2, kv=2, dim=32, vdim=32, conv=4, ff=64)],
}


@pytest.mark.parametrize("name", sorted(ALONE))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_each_mixer_alone(name, dtype):
    cfg = config(ALONE[name])
    m, o = build(cfg, seed=3, dtype=dtype)
    ids = toks(40, cfg["vocab"])
    got, resid = m.forward_rows(ids[None], 0, list(range(40)), want_residual=True)
    want = o.run(ids)
    assert resid.shape == (1, 40, cfg["width"])
    assert err(got, want) < (FP32_BAR if dtype == "float32" else BF16_BAR)
    m.close()


def test_no_side_input_and_plain_residual():
    cfg = config([lightning(), attn(), delta()], side=0, mult=1.0)
    m, o = build(cfg, seed=4)
    ids = toks(24, cfg["vocab"])
    assert err(m.forward_rows(ids[None], 0, list(range(24))), o.run(ids)) < FP32_BAR
    m.close()


MIXED = [lightning(ff=0), attn(ff=96), delta(ff=0), lightning(heads=4, dim=8, vdim=16, decay=(0.6, 0.9, 0.97, 0.999)), attn(heads=2, kv=1, dim=32, scale=0.2)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_then_token_by_token_and_portions(dtype):
    cfg = config(MIXED)
    m, o = build(cfg, seed=5, dtype=dtype, max_seq_len=160)
    bar = FP32_BAR if dtype == "float32" else BF16_BAR
    n = 150
    ids = toks(n, cfg["vocab"], seed=6)
    want = o.run(ids)
    whole = m.forward_rows(ids[None], 0, list(range(n)))
    assert err(whole, want) < bar
    # every token alone, from the first one
    one = np.stack([m.forward(ids[None, t:t + 1], t)[0] for t in range(n)])
    assert err(one, want) < bar
    # portions of changing size, down to two tokens and one
    for sizes in ([37, 3, 2, 2], [2], [64, 1, 5, 2, 31]):
        pos, i, rows = 0, 0, []
        while pos < n:
            c = min(sizes[i % len(sizes)], n - pos)
            i += 1
            rows.append(m.forward_rows(ids[None, pos:pos + c], pos, list(range(c))))
            pos += c
        got = np.concatenate(rows)
        assert err(got, want) < bar
        if dtype == "float32":  # the recurrences run the same chain however the prompt is cut
            assert err(got, whole) < 2e-6
    m.close()


def test_long_decoding_matches_the_oracle():
    cfg = config([delta(conv=4), lightning(decay=(0.9, 0.9995)), attn()], width=48)
    m, o = build(cfg, seed=7, max_seq_len=400)
    ids = toks(380, cfg["vocab"], seed=8)
    want = o.run(ids)
    m.forward_rows(ids[None, :20], 0, [])
    got = np.stack([m.forward(ids[None, t:t + 1], t)[0] for t in range(20, 380)])
    assert err(got, want[20:]) < FP32_BAR
    m.close()


def test_batch_rows_equal_single_sequences_and_slots_are_reused():
    cfg = config(MIXED)
    t = random_model(cfg, 9)
    m, o = build(cfg, tensors=t, max_seq_len=64, max_batch_size=3)
    ids = np.stack([toks(30, cfg["vocab"], seed=s) for s in (10, 11, 12)])
    batch = m.forward_rows(ids[:, :25], 0, list(range(75)))
    step = m.forward(ids[:, 25:26], 25)
    for b in range(3):
        want = o.run(ids[b, :26])
        assert err(batch[b * 25:(b + 1) * 25], want[:25]) < FP32_BAR
        assert err(step[b], want[25]) < FP32_BAR
    # slot 0 held sequence 0 up to position 26; a new sequence starting there must not see any of it
    again = m.forward_rows(ids[2:3, :30], 0, list(range(30)))
    assert err(again, o.run(ids[2])) < FP32_BAR
    # and continuing a slot anywhere but at its own position is refused
    with pytest.raises(RuntimeError):
        m.forward(ids[:1, :1], 7)
    m.close()


def test_far_key_dominates_attention():
    """One early key is made to match every later query far better than the rest: its value must come through
    hundreds of tokens later, in a prompt and in decoding."""
    cfg = config([attn(heads=2, kv=1, dim=16, scale=4.0)], width=32, vocab=50, side=0)
    t = random_model(cfg, 13)
    t["l0.mix.q"] = t["l0.mix.q"] * 3.0
    t["l0.mix.k"] = t["l0.mix.k"] * 3.0
    m, o = build(cfg, tensors=t, max_seq_len=700)
    ids = toks(650, 50, seed=14)
    want = o.run(ids)
    got = m.forward_rows(ids[None, :600], 0, list(range(600)))
    assert err(got, want[:600]) < FP32_BAR
    tail = np.stack([m.forward(ids[None, i:i + 1], i)[0] for i in range(600, 650)])
    assert err(tail, want[600:]) < FP32_BAR
    m.close()


def test_slow_decay_remembers_the_first_token():
    cfg = config([lightning(heads=2, dim=8, vdim=8, decay=(1.0, 0.9999))], width=32, vocab=50, side=0)
    m, o = build(cfg, seed=15, max_seq_len=600)
    ids = toks(520, 50, seed=16)
    want = o.run(ids)
    got = np.concatenate([m.forward_rows(ids[None, :500], 0, list(range(500))),
                          np.stack([m.forward(ids[None, i:i + 1], i)[0] for i in range(500, 520)])])
    assert err(got, want) < FP32_BAR
    S, _ = m.read_state(0)
    st = o.new_state()
    for tkn in ids:
        o.step(int(tkn), st)
    assert np.allclose(S, st[0]["S"], rtol=2e-4, atol=2e-4)
    m.close()


ODD = {
    # sizes the tiled kernels do not take, and values the usual configs make equal or 1
    "head_24": config([attn(heads=3, kv=1, dim=24, scale=0.5, ff=50)], width=72, vocab=61, side=5),
    "width_not_8": config([lightning(heads=1, dim=12, vdim=20, decay=(0.8,)), attn(heads=2, kv=2, dim=16, scale=1.0)], width=44, vocab=33, side=3),
    "width_not_4": config([delta(heads=3, kv=1, dim=10, vdim=6, conv=2), attn(heads=1, kv=1, dim=48, scale=0.05)], width=30, vocab=40, side=7),
    "one_tap_big_key": config([delta(heads=2, kv=1, dim=300, vdim=4, conv=1, ff=24)], width=40, vocab=25, side=0),
    "many_taps": config([delta(heads=1, kv=1, dim=8, vdim=40, conv=7)], width=24, vocab=25, side=2, mult=1.0, eps=1e-3),
}


@pytest.mark.parametrize("name", sorted(ODD))
def test_odd_sizes(name):
    cfg = ODD[name]
    m, o = build(cfg, seed=17)
    ids = toks(33, cfg["vocab"], seed=18)
    want = o.run(ids)
    got = np.concatenate([m.forward_rows(ids[None, :20], 0, list(range(20))), m.forward_rows(ids[None, 20:22], 20, [0, 1]),
                          np.stack([m.forward(ids[None, i:i + 1], i)[0] for i in range(22, 33)])])
    assert err(got, want) < FP32_BAR
    m.close()


def test_convolution_tail_and_state_after_short_portions():
    cfg = config([delta(heads=2, kv=2, dim=8, vdim=8, conv=4)], width=32, vocab=30, side=0)
    m, o = build(cfg, seed=19)
    ids = toks(9, 30, seed=20)
    for lo, hi in ((0, 1), (1, 3), (3, 4), (4, 9)):  # portions shorter than the convolution
        m.forward_rows(ids[None, lo:hi], lo, [])
    st = o.new_state()
    for tkn in ids:
        o.step(int(tkn), st)
    S, tail = m.read_state(0)
    want_tail = np.concatenate([st[0][f"mix.{n}.hist"] for n in "qkv"], axis=1).T  # [channels, taps - 1]
    assert np.allclose(tail, want_tail, rtol=1e-5, atol=1e-5)
    assert np.allclose(S, st[0]["S"], rtol=1e-4, atol=1e-5)
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_library_loop(dtype):
    cfg = config(MIXED)
    m, o = build(cfg, seed=21, dtype=dtype, max_seq_len=96, max_batch_size=2)
    prompts = np.stack([toks(12, cfg["vocab"], seed=s) for s in (22, 23)])
    lazy = np.concatenate(list(m.generate(prompts, 40)), axis=1)
    bulk = m.generate_all(prompts, 40)
    assert np.array_equal(lazy, bulk)
    # teacher-forced check: every emitted token is the oracle's argmax for the same prefix, unless the oracle's
    # top two are closer than the mode's error bar
    margin = 1e-3 if dtype == "float32" else 0.2
    for b in range(2):
        seq = np.concatenate([prompts[b], bulk[b]])
        lg = o.run(seq[:-1])
        for i in range(40):
            row = lg[11 + i]
            top = np.sort(row)[-2:]
            if top[1] - top[0] > margin * np.std(row):
                assert int(np.argmax(row)) == int(bulk[b, i]), f"sequence {b}, new token {i}"
    m.close()


def test_registry_and_checkpoint_folder(tmp_path):
    import json
    import struct
    from llama3_np_b200.models import load_model
    cfg = config([lightning(), attn()], width=32, vocab=41, side=4)
    t = random_model(cfg, 24)
    header, blob, off = {}, b"", 0
    for k, v in t.items():
        raw = (np.asarray(v, np.float32).view(np.uint32) >> 16).astype("<u2").tobytes()  # exact: values sit on the bf16 grid
        header[k] = {"dtype": "BF16", "shape": list(v.shape), "data_offsets": [off, off + len(raw)]}
        blob += raw
        off += len(raw)
    hj = json.dumps(header).encode()
    (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", len(hj)) + hj + blob)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    m = load_model(str(tmp_path), dtype="float32", max_seq_len=32)
    ids = toks(16, 41, seed=25)
    assert err(m.forward_rows(ids[None], 0, list(range(16))), OracleRisalix(cfg, t).run(ids)) < FP32_BAR
    m.close()


def test_trace_runner_replays_a_trace(tmp_path):
    """bin/trace_run as a user runs it: a checkpoint folder, steps on standard input, logits files out - two requests
    after one another through the same slot, portions cut in odd places and longer than one forward call."""
    import json
    import os
    import subprocess
    import sys
    from conftest import ROOT
    from test_risalix_cpu import write_safetensors
    cfg = config([lightning(), attn(ff=48), delta()], width=32, vocab=41, side=4)
    t = random_model(cfg, 26)
    write_safetensors(tmp_path / "model.safetensors", t)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    o = OracleRisalix(cfg, t)
    reqs = {"a": toks(23, 41, seed=27), "b": toks(9, 41, seed=28)}
    want = {k: o.run(v) for k, v in reqs.items()}
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
    assert not (out / f"{n}.f32").exists()


def test_generate_command_prints_the_loop_s_tokens(tmp_path):
    """bin/generate on a checkpoint folder: two prompts from a file as one batch, the printed ids are the ones the
    model's own greedy loop gives in-process."""
    import json
    import os
    import subprocess
    import sys
    from conftest import ROOT
    from llama3_np_b200.models import load_model
    from test_risalix_cpu import write_safetensors
    cfg = config([delta(heads=2, kv=1), attn(ff=40), lightning()], width=32, vocab=47, side=4)
    write_safetensors(tmp_path / "model.safetensors", random_model(cfg, 29))
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    prompts = np.stack([toks(7, 47, seed=s) for s in (30, 31)])
    (tmp_path / "prompts.txt").write_text("\n".join(" ".join(str(int(x)) for x in p) for p in prompts) + "\n")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "generate"), "--model", str(tmp_path), "--dtype", "float32",
                        "--batch-file", str(tmp_path / "prompts.txt"), "--new", "12"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    printed = np.array([[int(x) for x in line.split()] for line in r.stdout.strip().splitlines()[-2:]])
    m = load_model(str(tmp_path), dtype="float32", max_seq_len=19, max_batch_size=2)
    assert np.array_equal(printed, m.generate_all(prompts, 12))
    m.close()


@pytest.mark.parametrize("dim,vdim", [(64, 64), (128, 192), (64, 128)])
def test_long_prompts_of_decay_linear_layers_run_chunk_parallel(dim, vdim):
    """Prompts of 128 tokens and more take the chunk-parallel form of the fixed-decay recurrence for key sizes 64 / 128:
    against the token-by-token oracle with a last chunk that is not full, a portion that continues from a state,
    a fast and a very slow decay, two sequences of a batch, and decoding from the state it leaves."""
    cfg = config([lightning(heads=2, dim=dim, vdim=vdim, decay=(0.35, 0.9997), ff=0), attn(), lightning(heads=1, dim=dim, vdim=vdim, decay=(0.93,))],
                 width=64, vocab=59, side=0)
    t = random_model(cfg, 33)
    m, o = build(cfg, tensors=t, max_seq_len=520, max_batch_size=2)
    ids = np.stack([toks(500, 59, seed=s) for s in (34, 35)])
    want = [o.run(ids[b]) for b in range(2)]
    # 301 tokens (4 full chunks + 45), then 150 more from that state (chunked again), then short portions and single tokens
    got = [m.forward_rows(ids[:, :301], 0, list(range(2 * 301))).reshape(2, 301, -1),
           m.forward_rows(ids[:, 301:451], 301, list(range(2 * 150))).reshape(2, 150, -1),
           m.forward_rows(ids[:, 451:480], 451, list(range(2 * 29))).reshape(2, 29, -1)]
    got += [m.forward(ids[:, i:i + 1], i)[:, None, :] for i in range(480, 500)]
    got = np.concatenate(got, axis=1)
    for b in range(2):
        assert err(got[b], want[b]) < FP32_BAR
    S, _ = m.read_state(0, slot=1)
    st = o.new_state()
    for tkn in ids[1]:
        o.step(int(tkn), st)
    assert np.abs(S - st[0]["S"]).max() < 2e-5 * np.abs(st[0]["S"]).max()  # the slow head's state grows to hundreds
    # the same prompt token by token (the sequential kernel) gives the same logits to fp32 rounding
    one = m.forward_rows(ids[:1, :127], 0, list(range(127)))
    one = np.concatenate([one, m.forward_rows(ids[:1, 127:254], 127, list(range(127)))])
    assert err(one, got[0, :254]) < 2e-5
    m.close()


def test_unequal_prompts_are_bucketed_by_length_and_match_each_alone():
    """`generate_ragged`: five prompts of three lengths with two sequence slots - buckets of one length, split where a
    bucket is larger than the batch; every prompt yields what it yields alone, in the caller's order, and stops at EOS."""
    cfg = config(MIXED)
    t = random_model(cfg, 36)
    m, _ = build(cfg, tensors=t, max_seq_len=64, max_batch_size=2)
    lens = [9, 4, 9, 17, 9]
    prompts = [toks(n, cfg["vocab"], seed=40 + i) for i, n in enumerate(lens)]
    got = m.generate_ragged(prompts, 14)
    assert [len(g) for g in got] == [14] * 5
    for p, g in zip(prompts, got):
        assert np.array_equal(g, m.generate_all(p[None], 14)[0])
    eos = int(got[3][5])
    cut = m.generate_ragged(prompts, 14, eos_id=eos)
    first = int(np.argmax(got[3] == eos))
    assert np.array_equal(cut[3], got[3][: first + 1])
    with pytest.raises(ValueError):
        m.generate_ragged([prompts[0], []], 3)
    m.close()
