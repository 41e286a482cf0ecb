"""CPU suite of the Rakelorn family: the config reader, the order of layer runs, and the NumPy statement of the
design against hand-made cases (router, rotation, token shift, recurrence) and against itself (one-token steps
with carried state against a whole run)."""
import json

import numpy as np
import pytest

from llama3_np_b200.rakelorn import stack_config
from llama3_np_b200.stack import LATENT, MINGRU
from oracle import ref_rakelorn as R

CFG = {
    "architecture": "Rakelorn", "vocab": 53, "width": 40, "norm": {"eps": 1e-4}, "embedding": {"scale": 2.5},
    "loop": {"start": 1, "stop": 2, "times": 3},
    "layers": [
        {"type": "latent_attention",
         "mixer": {"heads": 3, "dim": 8, "rot_dim": 4, "vdim": 6, "q_rank": 12, "kv_rank": 20, "scale": 0.25,
                   "rot": {"base": 777.0, "dims": 4}},
         "mlp": {"kind": "moe", "expert": {"ff": 10},
                 "router": {"experts": 5, "top": 2, "identity": 1, "scale": 1.25, "groups": {"count": 3, "keep": 2}}}},
        {"type": "mingru", "mixer": {"width": 28}, "mlp": None},
    ],
}


def test_config_reader_takes_every_size_from_the_config():
    sc = stack_config(CFG, max_seq_len=77, max_batch_size=3, dtype="bfloat16")
    assert (sc.width, sc.vocab, sc.max_seq_len, sc.max_batch_size, sc.dtype) == (40, 53, 77, 3, "bfloat16")
    assert sc.norm_input and sc.norm_scalar and sc.token_shift and not sc.norm_one_plus
    assert sc.norm_eps == pytest.approx(1e-4) and sc.embed_scale == pytest.approx(2.5) and sc.loop == (1, 2, 3)
    la, gr = sc.layers
    assert (la.mixer, la.heads, la.dim, la.rot_dim, la.rot_dims, la.vdim, la.q_rank, la.kv_rank) == (LATENT, 3, 8, 4, 4, 6, 12, 20)
    assert la.scale == pytest.approx(0.25) and la.rot_base == pytest.approx(777.0)
    assert (la.ff, la.experts, la.top, la.identity, la.groups, la.groups_keep) == (10, 5, 2, 1, 3, 2)
    assert la.router_scale == pytest.approx(1.25)
    assert (gr.mixer, gr.heads, gr.dim, gr.vdim, gr.ff, gr.experts) == (MINGRU, 1, 28, 1, 0, 0)
    plain = json.loads(json.dumps(CFG))
    del plain["loop"]
    del plain["layers"][0]["mlp"]["router"]["groups"]
    del plain["layers"][0]["mlp"]["router"]["identity"]
    sc = stack_config(plain)
    assert sc.loop is None and (sc.layers[0].groups, sc.layers[0].groups_keep, sc.layers[0].identity) == (1, 1, 0)
    bad = json.loads(json.dumps(CFG))
    bad["layers"][1]["type"] = "hyena"
    with pytest.raises(ValueError):
        stack_config(bad)
    bad = json.loads(json.dumps(CFG))
    bad["layers"][0]["mlp"]["kind"] = "dense"
    with pytest.raises(ValueError):
        stack_config(bad)


def test_registry_knows_the_architecture():
    from llama3_np_b200.models import ARCHITECTURES
    assert "Rakelorn" in ARCHITECTURES


def test_layer_runs_order():
    runs = R.layer_runs(CFG)
    assert [(r[0], r[1]) for r in runs] == [(0, None), (1, 0), (1, 1), (1, 2)]
    assert [r[2] for r in runs] == [False, True, True, True]
    two = dict(CFG, loop={"start": 0, "stop": 2, "times": 2})
    assert [(r[0], r[2]) for r in R.layer_runs(two)] == [(0, True), (1, False), (0, True), (1, False)]
    assert [r[0] for r in R.layer_runs({"layers": [0, 0, 0]})] == [0, 1, 2]


def test_rotation_is_a_rotation_of_adjacent_pairs():
    v = np.arange(1.0, 9.0)
    r = R.rotate_pairs(v, 5, 4, 100.0)
    assert np.allclose(r[4:], v[4:])  # entries past `dims` pass unchanged
    a0, a1 = 5.0, 5.0 * 100.0 ** (-0.5)
    assert np.allclose(r[:2], [np.cos(a0) - 2 * np.sin(a0), 2 * np.cos(a0) + np.sin(a0)])
    assert np.allclose(r[2:4], [3 * np.cos(a1) - 4 * np.sin(a1), 4 * np.cos(a1) + 3 * np.sin(a1)])
    # the product of two rotated vectors depends on the distance of their positions only
    q, k = np.random.default_rng(0).standard_normal((2, 6))
    d1 = R.rotate_pairs(q, 40, 6, 50.0) @ R.rotate_pairs(k, 33, 6, 50.0)
    d2 = R.rotate_pairs(q, 107, 6, 50.0) @ R.rotate_pairs(k, 100, 6, 50.0)
    assert d1 == pytest.approx(d2)
    assert np.allclose(R.rotate_pairs(v, 0, 8, 10.0), v)


def test_token_shift_uses_the_unshifted_previous_input():
    st = {}
    mu = np.array([0.0, 1.0, 0.5])
    a = R.token_shift(np.array([1.0, 2.0, 3.0]), mu, st)
    assert np.allclose(a, [1.0, 0.0, 1.5])  # zeros ahead of the first token
    b = R.token_shift(np.array([5.0, 6.0, 7.0]), mu, st)
    assert np.allclose(b, [5.0, 2.0, 5.0])  # the previous h as it was before its own shift


def test_router_masks_groups_with_minus_infinity_and_weighs_by_the_plain_score():
    W = np.eye(6)
    P = {"mlp.router": W, "mlp.correction": np.array([-5.0, -5.0, -4.0, -4.2, -9.0, -9.0])}
    h = np.log(np.array([0.05, 0.05, 0.1, 0.1, 0.4, 0.3]))  # softmax(h) = these scores
    rc = {"experts": 4, "identity": 2, "top": 3, "scale": 2.0, "groups": {"count": 3, "keep": 1}}
    chosen, w = R.route(h, P, rc)
    # every choice score is negative; group 1 (slots 2, 3) has the largest best choice; with only two eligible slots
    # the third pick falls on a masked slot (minus infinity: the lowest index), never on a "zero"
    assert list(chosen[:2]) == [2, 3]
    assert np.allclose(w[:2], [0.2, 0.2])
    rc["groups"] = {"count": 3, "keep": 2}
    chosen, w = R.route(h, P, rc)
    assert list(chosen) == [2, 3, 0] and np.allclose(w, [0.2, 0.2, 0.1])
    rc = {"experts": 4, "identity": 2, "top": 2, "scale": 1.0}
    P["mlp.correction"] = np.zeros(6)
    chosen, w = R.route(h, P, rc)
    assert list(chosen) == [4, 5] and np.allclose(w, [0.4, 0.3])
    y = R.moe(np.arange(6.0), {**P, "mlp.router": np.zeros((6, 6)), "mlp.correction": np.array([0, 0, 0, 0, 1.0, 2.0])},
              {"expert": {"ff": 1}, "router": rc})
    assert np.allclose(y, np.arange(6.0) * (2.0 / 6.0))  # two identity slots: the input, weighted


def test_mingru_candidate_and_state():
    P = {"mix.z": np.zeros((2, 2)), "mix.z.b": np.array([0.0, 50.0]), "mix.x": np.eye(2), "mix.x.b": np.zeros(2),
         "mix.g": np.zeros((2, 2)), "mix.o": np.eye(2)}
    st = {}
    R.mingru_step(np.array([2.0, -1.0]), P, {"width": 2}, st)
    # z = (1/2, ~1): S = z * cand with cand = u + 1/2 above zero and sigmoid(u) below
    assert np.allclose(st["S"], [0.5 * 2.5, 1.0 / (1.0 + np.e)])
    R.mingru_step(np.array([0.0, 0.0]), P, {"width": 2}, st)
    assert np.allclose(st["S"], [0.5 * 1.25 + 0.5 * 0.5, 0.5])


def test_steps_with_carried_state_equal_a_whole_run():
    t = R.random_model(CFG, 3)
    ids = np.random.default_rng(4).integers(0, 53, 17)
    o = R.OracleRakelorn(CFG, t)
    whole, res = o.run(ids, want_residual=True)
    assert res.shape == (4, 17, 40)
    o.reset()
    parts = np.concatenate([o.run(ids[:5]), o.run(ids[5:6]), o.run(ids[6:])])
    assert np.allclose(parts, whole)
    o.reset()
    assert not np.allclose(o.run(ids[1:])[0], whole[1])  # the first token is part of every later answer
