"""CPU suite of the layer-list decoder family: the checkpoint reader, the config reader, the slot table, the
registry's refusal of unknown architectures, and the NumPy statement of the design against itself (state carried
across calls, one-token steps against a whole run)."""
import json
import struct

import numpy as np
import pytest

from llama3_np_b200.risalix import stack_config
from llama3_np_b200.stack import DECAY_LINEAR, GATED_DELTA, SOFTMAX, SlotTable
from llama3_np_b200.utils import read_safetensors
from oracle.ref_risalix import OracleRisalix, random_model

CFG = {
    "architecture": "Risalix", "vocab": 53, "width": 40, "residual_mult": 0.7, "norm": {"eps": 1e-4},
    "token_side": {"dim": 6},
    "layers": [
        {"type": "lightning", "mixer": {"heads": 2, "dim": 8, "vdim": 12, "decay": [0.5, 0.99]}, "mlp": None},
        {"type": "channel_delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 4, "conv": 3}, "mlp": {"kind": "dense", "ff": 24}},
        {"type": "attention", "mixer": {"heads": 6, "kv_heads": 2, "dim": 8, "vdim": 8, "scale": 0.2}, "mlp": None},
    ],
}


def write_safetensors(path, tensors, int_tables=()):
    header, blob, off = {}, b"", 0
    for k, v in tensors.items():
        if k in int_tables:
            raw, kind = np.asarray(v, "<i4").tobytes(), "I32"
        else:
            raw, kind = (np.asarray(v, np.float32).view(np.uint32) >> 16).astype("<u2").tobytes(), "BF16"
        header[k] = {"dtype": kind, "shape": list(np.shape(v)), "data_offsets": [off, off + len(raw)]}
        blob += raw
        off += len(raw)
    hj = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + blob)


def test_safetensors_reader_round_trip(tmp_path):
    t = random_model(CFG, 1)
    t["table"] = np.arange(12, dtype=np.int32).reshape(3, 4)
    write_safetensors(tmp_path / "m.safetensors", t, int_tables=("table",))
    back = read_safetensors(tmp_path / "m.safetensors")
    assert set(back) == set(t)
    assert back["table"].dtype == np.int32 and np.array_equal(back["table"], t["table"])
    for k in t:
        if k != "table":
            assert back[k].dtype == np.float32 and np.array_equal(back[k], t[k].astype(np.float32)), k


def test_config_reader_takes_every_size_from_config_or_shapes():
    t = random_model(CFG, 2)
    sc = stack_config(CFG, {k: v.shape for k, v in t.items()}, max_seq_len=77, max_batch_size=3, dtype="bfloat16")
    assert (sc.width, sc.vocab, sc.side_dim, sc.max_seq_len, sc.max_batch_size, sc.dtype) == (40, 53, 6, 77, 3, "bfloat16")
    assert sc.norm_eps == pytest.approx(1e-4) and sc.residual_mult == pytest.approx(0.7)
    lin, dlt, att = sc.layers
    assert (lin.mixer, lin.heads, lin.dim, lin.vdim, list(lin.decay), lin.ff) == (DECAY_LINEAR, 2, 8, 12, [0.5, 0.99], 0)
    assert (dlt.mixer, dlt.heads, dlt.kv_heads, dlt.conv_taps, dlt.ff) == (GATED_DELTA, 4, 2, 3, 24)
    assert dlt.rank_decay == t["l1.mix.a1"].shape[0] and dlt.rank_gate == t["l1.mix.g1"].shape[0]
    assert (att.mixer, att.heads, att.kv_heads, att.dim, att.scale) == (SOFTMAX, 6, 2, 8, pytest.approx(0.2))
    one = json.loads(json.dumps(CFG))
    one["layers"][0]["mixer"]["decay"] = 0.9  # a single number serves every head
    del one["token_side"]
    sc1 = stack_config(one, {k: v.shape for k, v in t.items()})
    assert list(sc1.layers[0].decay) == [0.9, 0.9] and sc1.side_dim == 0
    bad = json.loads(json.dumps(CFG))
    bad["layers"][0]["mixer"]["decay"] = [0.5]
    with pytest.raises(ValueError):
        stack_config(bad, None)
    bad = json.loads(json.dumps(CFG))
    bad["layers"][0]["type"] = "hyena"
    with pytest.raises(ValueError):
        stack_config(bad, None)
    bad = json.loads(json.dumps(CFG))
    bad["layers"][1]["mlp"]["kind"] = "experts"
    with pytest.raises(ValueError):
        stack_config(bad, None)


def test_slot_table_hands_back_freed_slots():
    s = SlotTable(2)
    assert s.acquire("a") == 0 and s.acquire("b") == 1 and s.acquire("a") == 0
    s.advance("a", 5)
    assert s.pos["a"] == 5
    with pytest.raises(RuntimeError):
        s.acquire("c")
    s.release("a")
    assert s.acquire("c") == 0 and s.pos["c"] == 0


def test_registry_refuses_unknown_architectures(tmp_path):
    from llama3_np_b200.models import load_model
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "Nope"}))
    with pytest.raises(ValueError):
        load_model(str(tmp_path))


def test_oracle_state_carries_across_calls():
    t = random_model(CFG, 3)
    o = OracleRisalix(CFG, t)
    ids = np.random.default_rng(4).integers(0, 53, 20)
    whole = o.run(ids)
    st = o.new_state()
    parts = np.concatenate([o.run(ids[:7], st), o.run(ids[7:9], st), o.run(ids[9:], st)])
    assert np.allclose(whole, parts, rtol=0, atol=1e-12)
    # the first token has no history at all: zero state, zero convolution tail, one key
    assert np.allclose(OracleRisalix(CFG, t).run(ids[:1]), whole[:1], atol=1e-12)
