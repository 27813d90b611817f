"""The slow float64 implementation of the Badepel architecture (tests/badepel_oracle.py) pinned on cases worked out by hand,
and its incremental form against its whole-sequence form.  No GPU."""
import math

import numpy as np

import badepel_oracle as O


def test_streams_read_and_write_by_hand():
    X = np.array([[[1.0, 2.0], [10.0, 20.0]]])          # one token, two streams, width 2
    a, b = np.array([0.5, 2.0]), np.array([1.0, -1.0])
    M = np.array([[1.0, 3.0], [0.0, 2.0]])              # [from, to]
    y = np.array([[100.0, 200.0]])
    assert np.allclose(O.streams_read(X, a), [[20.5, 41.0]])
    Xn = O.streams_write(X, y, M, b, 0.1)
    # stream 0 <- 1*X0 + 0*X1 + 0.1*1*y;  stream 1 <- 3*X0 + 2*X1 - 0.1*y
    assert np.allclose(Xn[0, 0], [11.0, 22.0]) and np.allclose(Xn[0, 1], [13.0, 26.0])
    # one stream with unit weights is the ordinary residual
    X1 = np.array([[[1.0, 2.0]]])
    assert np.allclose(O.streams_write(X1, y, np.ones((1, 1)), np.ones(1), 0.5)[0, 0], [51.0, 102.0])


def test_rms_has_eps_inside_the_root():
    assert np.allclose(O.rms(np.array([3.0, 4.0]), 0.5), np.array([3.0, 4.0]) / math.sqrt(12.5 + 0.5))


def test_rotation_of_neighbouring_pairs():
    rot = {"dims": 4, "base": 100.0}
    x = np.zeros((2, 1, 6))
    x[:, 0] = [1.0, 0.0, 0.0, 2.0, 5.0, 6.0]
    out = O.rotate_pairs(x, [0, 3], rot)
    assert np.allclose(out[0], x[0])                                    # position 0: nothing turns
    f1 = 100.0 ** (-2.0 / 4.0)
    assert np.allclose(out[1, 0, :2], [math.cos(3.0), math.sin(3.0)])   # (1, 0) by the angle 3 * 1
    assert np.allclose(out[1, 0, 2:4], [-2.0 * math.sin(3.0 * f1), 2.0 * math.cos(3.0 * f1)])
    assert np.allclose(out[1, 0, 4:], [5.0, 6.0])                       # beyond dims: untouched


def test_window_table():
    m = {"size": 3}
    assert [j for j in range(6) if O.in_window(4, j, m)] == [2, 3, 4]
    assert [j for j in range(6) if O.in_window(1, j, m)] == [0, 1]
    assert [j for j in range(6) if O.in_window(4, j, None)] == [0, 1, 2, 3, 4]
    assert [j for j in range(6) if O.in_window(4, j, {"size": 1})] == [4]


def test_softmax_with_a_zero_entry_that_has_no_value():
    assert np.allclose(O.zero_sink_softmax(np.array([0.0])), [0.5])
    assert np.allclose(O.zero_sink_softmax(np.array([math.log(3.0)])), [0.75])
    p = O.zero_sink_softmax(np.array([-50.0, -60.0]))
    assert p.sum() < 1e-20                                  # everything goes to the extra entry
    p = O.zero_sink_softmax(np.array([800.0, 800.0]))       # no overflow
    assert np.allclose(p, [0.5, 0.5])


def test_soft_cap():
    assert np.allclose(O.soft_cap(np.array([0.0, 1e9]), 5.0), [0.0, 5.0])
    assert O.soft_cap(3.0, None) == 3.0


def test_convolution_continues_from_its_tail():
    rng = np.random.default_rng(0)
    u, w = rng.standard_normal((9, 3)), rng.standard_normal((3, 4))
    y, tail = O.causal_conv(u, w, np.zeros((3, 3)))
    assert np.allclose(y[0], w[:, 3] * u[0]) and np.allclose(y[1], w[:, 3] * u[1] + w[:, 2] * u[0])
    ya, ta = O.causal_conv(u[:5], w, np.zeros((3, 3)))
    yb, tb = O.causal_conv(u[5:], w, ta)
    assert np.allclose(np.concatenate([ya, yb]), y) and np.allclose(tb, tail) and np.allclose(tail, u[6:])
    # one tap: a scale per channel and no tail
    y1, t1 = O.causal_conv(u, w[:, :1], np.zeros((0, 3)))
    assert np.allclose(y1, u * w[:, 0]) and t1.shape == (0, 3)


def test_linear_attention_write_decay_read():
    q = np.array([[[0.0, 0.0]], [[0.0, 0.0]], [[1.0, 1.0]]])
    k = np.array([[[1.0, 0.0]], [[0.0, 1.0]], [[0.0, 0.0]]])
    v = np.array([[[2.0]], [[3.0]], [[0.0]]])
    a = np.array([[[1.0, 1.0]], [[0.5, 0.25]], [[0.5, 0.25]]])
    S = np.zeros((1, 2, 1))
    o = O.gla_scan(q, k, v, a, S)
    # row 0 holds 2, decayed twice by 0.5; row 1 holds 3, decayed once by 0.25 (the decay acts before the token's own write)
    assert np.allclose(S[0, :, 0], [0.5, 0.75]) and np.allclose(o[2, 0], [1.25])


def test_delta_rule_replaces_what_a_key_holds():
    k = np.array([[[1.0, 0.0]], [[1.0, 0.0]], [[0.0, 1.0]]])
    v = np.array([[[2.0]], [[7.0]], [[4.0]]])
    q = k.copy()
    g, beta = np.ones((3, 1)), np.ones((3, 1))
    S = np.zeros((1, 2, 1))
    o = O.delta_scan(q, k, v, g, beta, S)
    assert np.allclose(o[:, 0, 0], [2.0, 7.0, 4.0])        # the read-out sees the token's own write
    assert np.allclose(S[0, :, 0], [7.0, 4.0])             # the second write replaced the first
    # half strength moves the row half way; a decay of one half first halves what is there
    S = np.array([[[2.0], [0.0]]])
    O.delta_scan(q[:1], k[:1], np.array([[[6.0]]]), np.array([[0.5]]), np.array([[0.5]]), S)
    assert np.allclose(S[0, :, 0], [1.0 + 0.5 * (6.0 - 1.0), 0.0])


def test_unit_length():
    assert np.allclose(O.unit(np.array([3.0, 4.0])), np.array([3.0, 4.0]) / math.sqrt(25.0 + 1e-6))


def one_layer(layer, **kw):
    cfg = O.make_config([layer], **kw)
    return cfg, O.random_weights(cfg, seed=3)


def test_decay_of_the_right_mixer_is_a_root_of_the_sigmoid():
    cfg, W = one_layer(O.parallel_layer(mlp=None, r_heads=1, r_dim=2, r_vdim=2, rank=1, tau=4.0))
    p = "l0.mix.right."
    W[p + "a1"][:] = 0.0
    W[p + "a2.b"][:] = [0.0, math.log(15.0)]        # sigmoid = 1/2 and 15/16
    W[p + "q"][:] = 0.0; W[p + "k"][:] = 0.0; W[p + "v"][:] = 0.0
    W[p + "k"][:, 0] = 1.0; W[p + "v"][:, 0] = 1.0; W[p + "q"][:, 1] = math.sqrt(2.0)
    h = np.zeros((3, cfg["width"]))
    h[0, 0] = 1.0      # token 0 writes 1 into both rows
    h[2, 1] = 1.0      # token 2 reads both rows
    st = {}
    W[p + "g"][:] = 0.0
    O.gla_mixer(h, {k: np.asarray(v, np.float64) for k, v in W.items()}, p, cfg["layers"][0]["mixer"]["right"], 1e-5, st)
    assert np.allclose(st["S"][0, :, 0], [0.5 ** (2 / 4.0), (15.0 / 16.0) ** (2 / 4.0)])


def test_router_takes_the_largest_logits_and_weighs_only_them():
    W = {"r.router": np.array([[1.0], [2.0], [3.0], [0.0]]), "r.router.b": np.array([0.0, 0.0, -2.5, 2.2])}
    idx, wts = O.route(np.array([[1.0]]), W, "r.", {"experts": 4, "top": 2})
    assert idx.tolist() == [[3, 1]]                          # logits 1, 2, 0.5, 2.2: the bias decides
    e = np.exp([2.2, 2.0])
    assert np.allclose(wts, [e / e.sum()])


def test_expert_clamps():
    W = {"e.gate": np.array([[1.0]]), "e.up": np.array([[1.0]]), "e.down": np.array([[1.0]])}
    big = O.expert(np.array([[10.0]]), W, "e.", 2.0)[0, 0]
    assert np.isclose(big, 2.0 * O.sigmoid(1.702 * 2.0) * 3.0)          # gate and up both held at the limit
    low = O.expert(np.array([[-10.0]]), W, "e.", 2.0)[0, 0]
    assert np.isclose(low, -10.0 * O.sigmoid(-17.02) * (-2.0 + 1.0))    # the gate has no lower limit, up stops at -limit


def test_shared_expert_has_its_own_limit():
    cfg, W = one_layer(O.delta_layer(mlp=O.moe(experts=2, top=1, ff=4, limit=0.01, shared=4, shared_limit=100.0)))
    W = {k: np.asarray(v, np.float64) for k, v in W.items()}
    h = np.random.default_rng(1).standard_normal((3, cfg["width"])) * 3.0
    f = cfg["layers"][0]["mlp"]
    with_shared = O.routed_ff(h, W, "l0.mlp.", f)
    alone = O.expert(h, W, "l0.mlp.shared.", 100.0)
    assert np.abs(with_shared - alone).max() < 0.2 * np.abs(alone).max()   # the routed experts are all but shut by their limit
    assert not np.allclose(O.expert(h, W, "l0.mlp.shared.", 0.01), alone)


def mixed_cfg():
    return O.make_config([
        O.delta_layer(mlp=O.dense()),
        O.parallel_layer(size=9),
        O.parallel_layer(heads=6, kv_heads=3, dim=8, vdim=12, conv=2, size=70, r_heads=2, r_dim=20, r_vdim=8, rank=8, mlp=None),
        O.delta_layer(heads=2, kv_heads=2, dim=20, vdim=20, conv=2, mlp=O.moe(experts=4, top=1, ff=16, shared=0)),
    ])


def test_whole_sequence_portions_and_single_tokens_agree():
    cfg = mixed_cfg()
    W = O.random_weights(cfg, seed=1)
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], 40).tolist()
    want, outs = O.forward(cfg, W, toks)
    for cuts in ([1] * 40, [2] * 20, [7, 1, 30, 2], [39, 1]):
        st, at, rows, lay = O.StepOracle(cfg, W), 0, [], []
        for c in cuts:
            lg, lo = st.step(toks[at:at + c])
            rows.append(lg); lay.append(lo); at += c
        assert np.allclose(np.concatenate(rows), want, atol=1e-9)
        assert np.allclose(np.concatenate(lay, 1), outs, atol=1e-9)


def test_a_model_without_stream_tensors_is_the_ordinary_residual():
    cfg = O.make_config([O.delta_layer(mlp=O.dense())], streams=1, residual_mult=0.5)
    W = O.random_weights(cfg, seed=2, hc=False)
    assert "l0.hc1.in" not in W
    toks = [3, 1, 4, 1, 5]
    lg, outs = O.forward(cfg, W, toks)
    Wd = {k: np.asarray(v, np.float64) for k, v in W.items()}
    x = Wd["embed"][toks]
    x = x + 0.5 * O.delta_mixer(O.rms(x, 1e-5) * Wd["l0.norm1"], Wd, "l0.mix.", cfg["layers"][0]["mixer"], 1e-5, {})
    x = x + 0.5 * O.dense_ff(O.rms(x, 1e-5) * Wd["l0.norm2"], Wd, "l0.mlp.")
    assert np.allclose(outs[0], x) and np.allclose(lg, (O.rms(x, 1e-5) * Wd["final.norm"]) @ Wd["head"].T)


def test_packaged_writer_and_slow_implementation_agree_on_names_and_shapes():
    from lmrs_b200 import model_dir as md
    cfg = md.badepel_config(64, 4, 50, streams=3, heads=4, kv_heads=2, head_dim=8, window=16, conv=3, gla_heads=2, gla_dim=8, gla_vdim=16, gla_rank=4,
                            delta_heads=4, delta_kv_heads=2, delta_dim=8, delta_vdim=16, ff=48, experts=3, top=2, expert_ff=24, shared_ff=16,
                            pattern=("delta", "parallel"), mlps=("dense", "moe", None))
    a = {n: tuple(s) for n, s, _ in md.badepel_tensors(cfg)}
    b = {n: tuple(s) for n, s, _ in O.tensor_table(cfg)}
    assert a == b
    assert "rank" not in md.written_badepel_config(cfg)["layers"][1]["mixer"]["right"]
    assert md.badepel_param_bytes(cfg) > 0 and md.badepel_matmul_flops_per_token(cfg) > 0 and md.badepel_mixer_flops(cfg, 64) > 0
