"""The slow Rupenex implementation of tests/rupenex_oracle.py against itself and against hand-made cases (no GPU):
whole-sequence arithmetic == the same fed in portions, and each mechanism on inputs whose answer is known in closed form.
The model-folder writer is checked against a byte-level read of its own file."""
import json
import math
import struct

import numpy as np

import rupenex_oracle as O


def small_cfg():
    return O.make_config([
        O.ssm_layer(),
        O.attention_layer(size=5, keep_first=2),
        O.ssm_layer(heads=2, vdim=8, state=6, groups=1, conv=1, norm_groups=1, mlp=O.moe(experts=3, identity=0, top=3, shared=0)),
        O.attention_layer(heads=2, kv_heads=2, size=0, rot_dims=0, mlp=None),
        O.attention_layer(heads=4, kv_heads=1, size=40, keep_first=0, factor=None, mlp=O.dense(ff=20, limit=0.5)),
    ], width=24, vocab=37)


def test_whole_sequence_equals_portions_and_single_tokens():
    cfg = small_cfg()
    W = O.random_weights(cfg, seed=3)
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], 19).tolist()
    whole, outs = O.forward(cfg, W, toks)
    assert outs.shape == (5, 19, 24)
    for cuts in ([1] * 19, [2, 3, 5, 7, 2], [18, 1]):
        inc, got, at = O.StepOracle(cfg, W), [], 0
        for c in cuts:
            got.append(inc.step(toks[at:at + c])[0])
            at += c
        assert np.allclose(np.concatenate(got), whole, rtol=0, atol=1e-9)


def test_layer_norm_takes_the_mean_off_and_has_no_bias():
    x = np.array([[1.0, 3.0, 5.0, 7.0]])
    got = O.layer_norm(x, np.array([1.0, 2.0, 1.0, 0.5]), 0.0)
    assert np.allclose(got[0], np.array([-3.0, -1.0, 1.0, 3.0]) / math.sqrt(5.0) * [1, 2, 1, 0.5])
    assert np.allclose(O.layer_norm(x + 100.0, np.ones(4), 0.0), O.layer_norm(x, np.ones(4), 0.0))
    assert np.allclose(O.layer_norm(np.full((1, 4), 9.0), np.ones(4), 1e-6), 0.0)   # eps sits inside the root
    assert np.allclose(O.rms(np.array([[3.0, 4.0]]), 0.0), [[3.0 / math.sqrt(12.5), 4.0 / math.sqrt(12.5)]])


def test_rotation_pairs_the_two_halves_and_divides_the_frequencies():
    rot = {"base": 100.0, "dims": 4, "scaling": {"factor": 2.0}}
    assert np.allclose(O.rot_freqs(rot), [0.5, 0.05])
    assert np.allclose(O.rot_freqs({"base": 100.0, "dims": 4}), [1.0, 0.1])
    z = np.arange(1.0, 7.0).reshape(1, 1, 6)
    r = O.rotate_halves(z, [3], rot)[0, 0]
    a0, a1 = 1.5, 0.15
    assert np.allclose(r, [1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
                           3 * math.cos(a0) + 1 * math.sin(a0), 4 * math.cos(a1) + 2 * math.sin(a1), 5, 6])
    assert np.allclose(O.rotate_halves(z, [0], rot), z)
    assert O.rotate_halves(z, [5], None) is z


def test_window_keeps_the_first_positions():
    mask = {"size": 3, "keep_first": 2}
    seen = [j for j in range(11) if O.visible(9, j, mask)]
    assert seen == [0, 1, 7, 8, 9]
    assert [j for j in range(11) if O.visible(2, j, mask)] == [0, 1, 2]
    assert [j for j in range(6) if O.visible(4, j, {"size": 2})] == [3, 4]
    assert [j for j in range(6) if O.visible(4, j, None)] == [0, 1, 2, 3, 4]


def test_the_sink_counts_once_in_the_denominator_and_has_no_value():
    w = O.sink_softmax(np.zeros(3), 0.0)
    assert np.allclose(w, 0.25) and math.isclose(w.sum(), 0.75)
    assert np.allclose(O.sink_softmax(np.zeros(3), None), 1.0 / 3.0)
    w = O.sink_softmax(np.array([1.0, 2.0]), 50.0)   # a large sink takes nearly all the weight away
    assert w.sum() < 1e-20
    w = O.sink_softmax(np.array([700.0, 701.0]), -700.0)   # no overflow either way
    assert np.allclose(w, [1 / (1 + math.e), math.e / (1 + math.e)])


def attention_weights(cfg_layer, n, width=8, seed=0, **edits):
    """one attention layer's mixer on random rows; returns (output rows, the weights W used)"""
    m = cfg_layer["mixer"]
    cfg = O.make_config([cfg_layer], width=width, vocab=11)
    W = O.random_weights(cfg, seed=seed)
    W.update(edits)
    h = np.random.default_rng(seed + 1).standard_normal((n, width))
    return O.attention_mixer(h, W, "l0.mix.", m, 1e-5, {}, 0), W, h, m


def test_attention_gate_reads_the_mixers_input_and_the_sink_shrinks_the_output():
    layer = O.attention_layer(heads=2, kv_heads=1, dim=4, vdim=4, size=0, rot_dims=0, mlp=None)
    out, W, h, m = attention_weights(layer, 1)
    # one token: its only key is its own, weight exp(s) / (exp(s) + exp(sink))
    q = O.rms((h @ W["l0.mix.q"].T).reshape(1, 2, 4), 1e-5) * W["l0.mix.q.norm"]
    k = O.rms((h @ W["l0.mix.k"].T).reshape(1, 1, 4), 1e-5) * W["l0.mix.k.norm"]
    v = (h @ W["l0.mix.v"].T).reshape(1, 1, 4)
    heads = []
    for hh in range(2):
        s = float(q[0, hh] @ k[0, 0]) * m["scale"]
        heads.append(math.exp(s) / (math.exp(s) + math.exp(W["l0.mix.sink"][hh])) * v[0, 0])
    want = (np.concatenate(heads) * O.sigmoid(h[0] @ W["l0.mix.g"].T)) @ W["l0.mix.o"].T
    assert np.allclose(out[0], want)


def test_causal_conv_continues_from_its_tail_and_adds_its_bias():
    rng = np.random.default_rng(1)
    x, w, b = rng.standard_normal((9, 3)), rng.standard_normal((3, 4)), rng.standard_normal(3)
    whole, tail = O.causal_conv(x, w, b, np.zeros((3, 3)))
    assert np.allclose(whole[0], x[0] * w[:, 3] + b) and np.allclose(whole[2], x[2] * w[:, 3] + x[1] * w[:, 2] + x[0] * w[:, 1] + b)
    a, t1 = O.causal_conv(x[:4], w, b, np.zeros((3, 3)))
    c, t2 = O.causal_conv(x[4:], w, b, t1)
    assert np.allclose(np.concatenate([a, c]), whole) and np.allclose(t2, tail) and np.allclose(tail, x[6:])
    one, _ = O.causal_conv(x, w[:, :1], b, np.zeros((0, 3)))
    assert np.allclose(one, x * w[:, 0] + b)


def test_state_space_scan_writes_reads_and_decays():
    # one head, two state rows, one value channel: B writes into a row, C reads it back, the decay is exp(-exp(A_log) dt)
    x = np.array([[[2.0]], [[0.0]], [[0.0]]])
    dt = np.array([[0.5], [1.0], [2.0]])
    Bm = np.array([[[1.0, 0.0]], [[0.0, 0.0]], [[0.0, 0.0]]])
    Cm = np.array([[[1.0, 0.0]], [[1.0, 0.0]], [[3.0, 5.0]]])
    S = np.zeros((1, 2, 1))
    y = O.ssm_scan(x, dt, np.array([math.log(0.25)]), Bm, Cm, np.array([10.0]), S)
    assert math.isclose(y[0, 0, 0], 0.5 * 2.0 + 10.0 * 2.0)        # written with weight dt, read at once, plus the skip
    assert math.isclose(y[1, 0, 0], 1.0 * math.exp(-0.25 * 1.0))
    assert math.isclose(y[2, 0, 0], 3.0 * math.exp(-0.25 * 3.0))   # decays multiply; the untouched row reads zero
    assert np.allclose(S[0, :, 0], [math.exp(-0.75), 0.0])
    # heads share the B and C of their group
    x = np.ones((1, 4, 1))
    Bm, Cm = np.array([[[1.0], [2.0]]]), np.array([[[1.0], [1.0]]])
    y = O.ssm_scan(x, np.ones((1, 4)), np.zeros(4), Bm, Cm, np.zeros(4), np.zeros((4, 1, 1)))
    assert np.allclose(y[0, :, 0], [1.0, 1.0, 2.0, 2.0])


def test_the_gate_comes_before_the_grouped_norm():
    y = np.array([[1.0, 2.0, 30.0, 40.0]])
    g = O.grouped_rms(y, 2, 0.0)
    assert np.allclose(g, [[1 / math.sqrt(2.5), 2 / math.sqrt(2.5), 30 / math.sqrt(1250.0), 40 / math.sqrt(1250.0)]])
    assert not np.allclose(g, O.grouped_rms(y, 1, 0.0))
    # the whole mixer on one token (empty state: y = (dt B.C + D) x), by hand
    m = O.ssm_layer(heads=2, vdim=2, state=3, groups=1, conv=2, norm_groups=2, mlp=None)["mixer"]
    cfg = O.make_config([{"type": "mamba2", "mixer": m, "mlp": None}], width=6, vocab=5)
    W = O.random_weights(cfg, seed=2)
    h = np.random.default_rng(3).standard_normal((1, 6))
    p = h @ W["l0.mix.in"].T
    z, xbc, dt = p[0, :4], p[0, 4:14], p[0, 14:]
    xbc = O.silu(xbc * W["l0.mix.conv"][:, 1] + W["l0.mix.conv.b"])
    x, Bv, Cv = xbc[:4].reshape(2, 2), xbc[4:7], xbc[7:10]
    dt = np.log1p(np.exp(dt + W["l0.mix.dt_bias"]))
    y = ((dt * float(Bv @ Cv) + W["l0.mix.D"])[:, None] * x).reshape(4)
    gated = y * z / (1.0 + np.exp(-z))
    want = (O.grouped_rms(gated[None], 2, 1e-5)[0] * W["l0.mix.norm"]) @ W["l0.mix.o"].T
    got = O.ssm_mixer(h, W, "l0.mix.", m, 1e-5, {})
    assert np.allclose(got[0], want)
    other = (O.grouped_rms(y[None], 2, 1e-5)[0] * z / (1.0 + np.exp(-z)) * W["l0.mix.norm"]) @ W["l0.mix.o"].T
    assert not np.allclose(got[0], other)


def test_dense_feed_forward_clamps_gate_from_above_and_up_from_both_sides():
    W = {"p.gate": np.array([[1.0]]), "p.up": np.array([[1.0]]), "p.down": np.array([[1.0]])}
    f = {"limit": 2.0}
    for v, g, u in ((1.0, 1.0, 1.0), (5.0, 2.0, 2.0), (-5.0, -5.0, -2.0)):
        want = g / (1.0 + math.exp(-1.702 * g)) * (u + 1.0)
        assert math.isclose(O.dense_ff(np.array([[v]]), W, "p.", f)[0, 0], want)
    assert math.isclose(O.dense_ff(np.array([[5.0]]), W, "p.", {})[0, 0], 5.0 / (1.0 + math.exp(-1.702 * 5.0)) * 6.0)


def test_router_softmax_runs_over_identity_experts_too_and_the_correction_only_chooses():
    r = {"experts": 2, "identity": 2, "top": 2}
    W = {"p.router": np.eye(4), "p.correction": np.array([0.0, 0.0, 0.0, 10.0])}
    h = np.array([[2.0, 1.0, 0.0, -5.0]])
    idx, w = O.route(h, W, "p.", r)
    s = np.exp(h[0]) / np.exp(h[0]).sum()
    assert idx[0].tolist() == [3, 0]   # output 3 wins through its correction only
    assert np.allclose(w[0], np.array([s[3], s[0]]) / (s[3] + s[0])) and math.isclose(w.sum(), 1.0)
    # identity experts return the input; the shared expert is added for every token
    W.update({"p.e0.up": np.zeros((3, 4)), "p.e0.down": np.zeros((4, 3)), "p.e1.up": np.zeros((3, 4)), "p.e1.down": np.zeros((4, 3))})
    f = {"router": r, "expert": {"ff": 3}}
    assert np.allclose(O.routed_ff(h, W, "p.", f), w[0, 0] * h)
    W.update({"p.shared.up": np.array([[1.0, 0, 0, 0], [0, 0, 0, 1.0]]), "p.shared.down": np.array([[1.0, 1.0]] * 4)})
    f["shared"] = {"ff": 2}
    assert np.allclose(O.routed_ff(h, W, "p.", f), w[0, 0] * h + 4.0)   # relu(2)^2 + relu(-5)^2
    assert np.allclose(O.expert(np.array([[3.0, 0, 0, -1.0]]), W, "p.shared."), 9.0)


def test_write_model_layout(tmp_path):
    cfg = small_cfg()
    W = O.random_weights(cfg, seed=4)
    d = O.write_model(str(tmp_path / "m"), cfg, W)
    raw = open(d + "/model.safetensors", "rb").read()
    n = struct.unpack("<Q", raw[:8])[0]
    hdr = json.loads(raw[8:8 + n])
    assert n % 8 == 0 and set(hdr) == set(W)
    e = hdr["l0.mix.conv"]
    assert e["dtype"] == "BF16" and e["shape"] == [4 * 10 + 2 * 2 * 12, 4]
    bits = np.frombuffer(raw[8 + n + e["data_offsets"][0]:8 + n + e["data_offsets"][1]], np.uint16)
    assert np.array_equal((bits.astype(np.uint32) << 16).view(np.float32).reshape(e["shape"]), W["l0.mix.conv"].astype(np.float32))
    assert hdr["l1.mlp.router"]["shape"] == [7, 24] and "l3.norm2" not in hdr and "l2.mlp.shared.up" not in hdr
    assert json.load(open(d + "/config.json"))["layers"][0]["type"] == "mamba2"


def test_the_packaged_writer_names_the_same_tensors():
    """lmrs_b200.model_dir (random models for benchmarks) and this file's table agree on names and shapes"""
    from lmrs_b200 import model_dir as md
    cfg = md.rupenex_config(48, 5, 90, heads=4, kv_heads=2, head_dim=8, window=12, keep_first=3, rot_dims=4, ssm_heads=3, ssm_vdim=16, state=10,
                            groups=1, conv=3, norm_groups=3, ff=40, experts=5, identity=1, top=2, expert_ff=24, shared_ff=32,
                            pattern=("mamba2", "attention"), mlps=("dense", "moe", None))
    assert [L["type"] for L in cfg["layers"]] == ["mamba2", "attention", "mamba2", "attention", "mamba2"]
    assert [(L["mlp"] or {}).get("kind") for L in cfg["layers"]] == ["dense", "moe", None, "dense", "moe"]
    a = {n: tuple(s) for n, s, _ in md.rupenex_tensors(cfg)}
    b = {n: tuple(s) for n, s, _ in O.tensor_table(cfg)}
    assert a == b
    # the chosen experts' share of the expert matrices, everything else once
    rest = sum(int(np.prod(s)) for n, s in a.items() if ".mlp.e" not in n and n != "embed")
    experts = sum(int(np.prod(s)) for n, s in a.items() if ".mlp.e" in n)
    assert md.rupenex_param_bytes(cfg) == int((rest + a["embed"][1] + experts * 2 / 6) * 2)
    W = O.random_weights(cfg, seed=1)
    logits, _ = O.forward(cfg, W, [1, 2, 3])
    assert logits.shape == (3, 90) and np.isfinite(logits).all()
