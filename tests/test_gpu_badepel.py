"""Badepel folder models on the GPU against the slow float64 implementation of tests/badepel_oracle.py.

Small random models (bf16-representable weights, so both operand modes load the same numbers) are written to a temporary
folder and opened through lmrs_b200.Transformer.open -- the entry point trace replay, forward, forward_argmax and
generate_greedy share.  float32 mode is held to 2e-4 of the logits' root mean square, bfloat16 mode to 4e-2.  For float32
the weights are drawn until no routing decision of the run is a close call.  In bfloat16 a run may legitimately take the
other expert where two logits are a hair apart (and a recurrent layer carries that on), so the bfloat16 comparisons against
the slow implementation use models whose routers choose all of their experts -- the weights still matter, no choice can
flip."""
import numpy as np
import pytest

import badepel_oracle as O

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-4, "bfloat16": 4e-2}
GAP = 1e-4
P, D = O.parallel_layer, O.delta_layer


def mixed_cfg(dtype="float32", **kw):
    """both mixers, both feed-forwards, a layer without one, grouped and ungrouped heads, windows shorter and longer than a key
    tile, sizes that are no powers of two and differ from each other; for bfloat16 every router chooses all of its experts"""
    ff = (lambda e, t, f, s: O.moe(e, t, f, shared=s)) if dtype == "float32" else (lambda e, t, f, s: O.moe(e, e, f, shared=s))
    return O.make_config([
        D(mlp=O.dense()),
        P(size=9, mlp=ff(5, 2, 24, 40)),
        P(heads=6, kv_heads=3, dim=8, vdim=12, conv=2, size=70, rot_dims=8, r_heads=2, r_dim=20, r_vdim=8, rank=8, mlp=None),
        D(heads=2, kv_heads=2, dim=20, vdim=20, conv=2, mlp=ff(4, 1, 16, 0)),
        P(heads=3, kv_heads=3, dim=16, vdim=8, conv=1, size=0, rot_dims=6, softcap=0.0, r_heads=1, r_dim=36, r_vdim=10, tau=1.0, mlp=O.dense(ff=30)),
    ], **kw)


def open_model(gpu_lib, tmp_path, cfg, W, dtype, max_tokens=256, name="m"):
    return gpu_lib.Transformer.open(O.write_model(str(tmp_path / name), cfg, W), dtype=dtype, max_tokens=max_tokens)


def tokens_for(cfg, n, seed=0):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


def weights_for(cfg, toks, seed=0, **kw):
    for s in range(seed, seed + 400, 7):
        W = O.random_weights(cfg, seed=s, **kw)
        if O.clear_choices(cfg, W, toks, GAP):
            return W
    raise AssertionError("no seed without a close routing decision")


def typical_row_close(got, want, tol):
    """the median row within tolerance and most rows too: a few may show an expert choice that flipped on a near-tie"""
    e = np.array([O.rel_rms(g, w) for g, w in zip(got, want)])
    return np.median(e) < tol and np.mean(e > tol) <= 0.35


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompt_logits_and_every_layer(gpu_lib, tmp_path, dtype):
    cfg = mixed_cfg(dtype)
    toks = tokens_for(cfg, 85)
    W = weights_for(cfg, toks, seed=1)
    want, outs = O.forward(cfg, W, toks)
    m = open_model(gpu_lib, tmp_path, cfg, W, dtype)
    assert m.args.model_type == gpu_lib.ModelType.BADEPEL and m.args.vocab_size == cfg["vocab"] and m.args.n_layers == 5
    m.set_option("keep_layers", 1)
    got = m.forward_tokens(toks, 0, list(range(85)))
    lo = m.layer_outputs(85)
    for li in range(5):   # the first layer that differs names the broken mechanism
        assert O.rel_rms(lo[li], outs[li]) < TOL[dtype], f"sum of the streams after layer {li}"
    assert O.rel_rms(got, want) < TOL[dtype]
    assert m.kernel_launches() > 0
    # the sums asked for per layer come from passes of their own over the streams: the logits are the same without them
    m.set_option("keep_layers", 0)
    assert np.array_equal(m.forward_tokens(toks, 0, list(range(85))), got)
    m.close()


# each mechanism alone: a one-layer model in which only that mechanism is not trivial, in shapes that take different branches
ALONE = {
    "delta": dict(layers=[D(mlp=None)]),
    "delta_one_tap": dict(layers=[D(conv=1, mlp=None)]),
    "delta_many_taps": dict(layers=[D(conv=7, mlp=None)]),
    "delta_ungrouped": dict(layers=[D(heads=3, kv_heads=3, mlp=None)]),
    "delta_one_kv_head": dict(layers=[D(heads=5, kv_heads=1, mlp=None)]),
    "delta_keys_over_two_lanes": dict(layers=[D(heads=2, kv_heads=1, dim=20, vdim=12, mlp=None)]),
    "delta_keys_over_several_lanes": dict(layers=[D(heads=2, kv_heads=2, dim=44, vdim=12, mlp=None)]),
    "delta_keys_over_half_a_warp": dict(layers=[D(heads=2, kv_heads=1, dim=72, vdim=6, mlp=None)]),
    "delta_keys_over_a_warp": dict(layers=[D(heads=2, kv_heads=2, dim=136, vdim=8, mlp=None)]),
    "delta_widest_keys": dict(layers=[D(heads=1, kv_heads=1, dim=264, vdim=6, mlp=None)]),
    "delta_wide_values": dict(layers=[D(heads=2, kv_heads=1, dim=8, vdim=136, mlp=None)]),
    "parallel": dict(layers=[P(mlp=None)]),
    "left_only": dict(layers=[P(right_scale=0.0, left_scale=1.0, mlp=None)]),
    "right_only": dict(layers=[P(right_scale=1.0, left_scale=0.0, mlp=None)]),
    "left_no_window": dict(layers=[P(size=0, mlp=None)]),
    "left_window_of_one": dict(layers=[P(size=1, mlp=None)]),
    "left_window_one_tile": dict(layers=[P(size=64, mlp=None)]),
    "left_window_tile_plus_one": dict(layers=[P(size=65, mlp=None)]),
    "left_window_longer_than_the_prompt": dict(layers=[P(size=500, mlp=None)]),
    "left_no_rotation": dict(layers=[P(rot_dims=0, mlp=None)]),
    "left_whole_head_rotated": dict(layers=[P(rot_dims=12, mlp=None)]),
    "left_no_cap": dict(layers=[P(softcap=0.0, scale=1.5, mlp=None)]),
    "left_cap_that_bites": dict(layers=[P(softcap=0.7, scale=3.0, mlp=None)]),
    "left_no_convolution": dict(layers=[P(conv=0, mlp=None)]),
    "left_one_tap": dict(layers=[P(conv=1, mlp=None)]),
    "left_many_taps": dict(layers=[P(conv=6, mlp=None)]),
    "left_one_kv_head": dict(layers=[P(heads=5, kv_heads=1, size=33, mlp=None)]),
    "left_ungrouped": dict(layers=[P(heads=3, kv_heads=3, dim=8, vdim=8, rot_dims=8, mlp=None)]),
    "left_many_heads_per_kv_head": dict(layers=[P(heads=20, kv_heads=1, dim=8, vdim=8, rot_dims=4, mlp=None)]),
    "left_wide_values": dict(layers=[P(heads=2, kv_heads=1, dim=8, vdim=72, size=40, rot_dims=2, mlp=None)]),
    "left_odd_head_sizes": dict(layers=[P(heads=3, kv_heads=1, dim=7, vdim=5, rot_dims=4, mlp=None)]),
    "right_one_head_tau_one": dict(layers=[P(r_heads=1, tau=1.0, mlp=None)]),
    "right_keys_over_several_lanes": dict(layers=[P(r_heads=2, r_dim=44, r_vdim=12, rank=16, mlp=None)]),
    "right_keys_over_a_warp": dict(layers=[P(r_heads=2, r_dim=136, r_vdim=8, rank=3, mlp=None)]),
    "right_wide_values": dict(layers=[P(r_heads=2, r_dim=8, r_vdim=136, mlp=None)]),
    "right_rank_one": dict(layers=[P(rank=1, mlp=None)]),
    "one_stream": dict(layers=[D(), P()], streams=1),
    "one_stream_unit_multiplier": dict(layers=[D(), P()], streams=1, residual_mult=1.0),
    "two_streams": dict(layers=[D(), P()], streams=2),
    "five_streams": dict(layers=[D(), P()], streams=5),
    "nine_streams": dict(layers=[D(), P()], streams=9),
    "dense_ff": dict(layers=[D(mlp=O.dense())]),
    "experts": dict(layers=[D(mlp=O.moe())]),
    "experts_top_one_no_shared": dict(layers=[D(mlp=O.moe(experts=4, top=1, shared=0))]),
    "experts_all_chosen": dict(layers=[D(mlp=O.moe(experts=3, top=3))]),
    "experts_that_clamp_hard": dict(layers=[D(mlp=O.moe(limit=0.1, shared_limit=0.05))]),
    "experts_many": dict(layers=[D(mlp=O.moe(experts=40, top=5, ff=8, shared=16))]),
    "odd_width": dict(layers=[D(heads=3, kv_heads=1, dim=10, vdim=6), P(dim=10, vdim=6, rot_dims=6, r_heads=3, r_dim=5, r_vdim=7)], width=27, vocab=33),
    # rows too long for the stream kernel to hold in registers between its passes
    "very_wide_rows": dict(layers=[D(heads=2, kv_heads=1, dim=8, vdim=8, mlp=O.moe(experts=2, top=2, ff=8, shared=8))], width=2056, vocab=20, streams=2),
}


@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mechanism_alone(gpu_lib, tmp_path, name):
    kw = dict(ALONE[name])
    cfg = O.make_config(kw.pop("layers"), **kw)
    toks = tokens_for(cfg, 70, seed=2)   # crosses one key-tile border
    W = weights_for(cfg, toks, seed=5, gain=2.0)
    want, _ = O.forward(cfg, W, toks)
    m = open_model(gpu_lib, tmp_path, cfg, W, "float32")
    got = m.forward_tokens(toks, 0, list(range(70)))
    assert O.rel_rms(got, want) < TOL["float32"]
    # and token by token through the decode step
    for i, t in enumerate(toks):
        lg = m.forward(t, i)
        if i in (0, 1, 2, 3, 63, 64, 65, 66, 67, 69):
            assert O.rel_rms(lg, want[i]) < TOL["float32"], f"decoded position {i}"
    m.close()


def test_a_model_without_stream_tensors(gpu_lib, tmp_path):
    """one stream and no read / write / mixing tensors: the ordinary residual with the multiplier"""
    cfg = O.make_config([D(), P()], streams=1, residual_mult=0.8)
    toks = tokens_for(cfg, 40, seed=2)
    W = O.random_weights(cfg, seed=6, hc=False)
    want, _ = O.forward(cfg, W, toks)
    cfg2 = dict(cfg)
    del cfg2["streams"]   # and the entry itself may be absent
    m = open_model(gpu_lib, tmp_path, cfg2, W, "float32")
    assert O.rel_rms(m.forward_tokens(toks, 0, list(range(40))), want) < TOL["float32"]
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_every_size_and_decoding_agree_with_the_whole_prompt(gpu_lib, tmp_path, dtype):
    cfg = mixed_cfg(dtype)
    n = 150
    toks = tokens_for(cfg, n, seed=3)
    W = weights_for(cfg, toks, seed=2, gain=1.5)
    want, _ = O.forward(cfg, W, toks)
    m = open_model(gpu_lib, tmp_path, cfg, W, dtype)
    for cuts in ([n], [2] * 8 + [3, 61, 2, 64, 1, 1, 1, 1], [63, 1, 64, 2, 20], [1] * 6 + [129, 2, 13], [127, 23]):
        assert sum(cuts) == n
        at, rows = 0, []
        for c in cuts:   # the same handle again and again: what an earlier schedule left in cache and state must not matter
            rows.append(m.forward_tokens(toks[at:at + c], at, list(range(c))))
            at += c
        assert O.rel_rms(np.concatenate(rows), want) < TOL[dtype], cuts
    # a long internal portion split by the library itself
    m.set_option("chunk_rows", 37)
    assert O.rel_rms(m.forward_tokens(toks, 0, list(range(n))), want) < TOL[dtype]
    m.close()


def test_portions_do_not_change_the_numbers_beyond_rounding(gpu_lib, tmp_path):
    """a position's logits from a whole prompt, from two-token portions and from single tokens differ by summation order only"""
    cfg = mixed_cfg()
    toks = tokens_for(cfg, 90, seed=4)
    W = weights_for(cfg, toks, seed=3)
    m = open_model(gpu_lib, tmp_path, cfg, W, "float32")
    whole = m.forward_tokens(toks, 0, list(range(90)))
    pairs = np.concatenate([m.forward_tokens(toks[i:i + 2], i, [0, 1]) for i in range(0, 90, 2)])
    singles = np.stack([m.forward(t, i).copy() for i, t in enumerate(toks)])
    assert O.rel_rms(pairs, whole) < 2e-5 and O.rel_rms(singles, whole) < 2e-5
    m.close()


def test_wanted_rows_in_any_order(gpu_lib, tmp_path):
    cfg = mixed_cfg()
    toks = tokens_for(cfg, 40)
    W = weights_for(cfg, toks, seed=4)
    want, _ = O.forward(cfg, W, toks)
    m = open_model(gpu_lib, tmp_path, cfg, W, "float32")
    idx = [39, 0, 17, 17, 5]
    assert O.rel_rms(m.forward_tokens(toks, 0, idx), want[idx]) < TOL["float32"]
    assert m.forward_tokens(toks, 0, []).shape == (0, cfg["vocab"])
    m.set_option("chunk_rows", 16)
    assert O.rel_rms(m.forward_tokens(toks, 0, idx), want[idx]) < TOL["float32"]
    m.close()


def private_channel(W, toks, dim=0):
    """an input dimension becomes private to some tokens: their embedding is large there, every other token's is zero (an RMS
    norm keeps a zero a zero)"""
    E = W["embed"]
    E[:, dim] = 0.0
    E[toks, dim] = 8.0
    for k in W:
        if k.endswith("norm1"):
            W[k][dim] = 1.0


def check_one_key_matters(gpu_lib, tmp_path, cfg, W, n, places, a_tok, b_tok, seen):
    """The last token (b) asks for the one earlier token (a) whose key matches it.  Where `seen(place)` says the key is visible,
    taking it away must move the slow implementation's answer a lot (the case has teeth); where it is not, the answer must not
    depend on it.  The library must agree in a prompt and in decoding."""
    m = open_model(gpu_lib, tmp_path, cfg, W, "float32", max_tokens=n + 8)
    for far in places:
        toks = [t if t < a_tok else 0 for t in tokens_for(cfg, n, seed=far)]
        toks[far], toks[n - 1] = a_tok, b_tok
        want, _ = O.forward(cfg, W, toks)
        toks2 = list(toks)
        toks2[far] = 0
        moved = O.rel_rms(O.forward(cfg, W, toks2)[0][n - 1], want[n - 1])
        if seen(far):
            assert moved > 100 * TOL["float32"], f"key at {far}: the case has no teeth ({moved})"
        else:
            assert moved < 1e-9, f"key at {far} should be invisible"
        got = m.forward_tokens(toks, 0, [n - 1])
        assert O.rel_rms(got[0], want[n - 1]) < TOL["float32"], f"key at {far} (prompt)"
        m.forward_tokens(toks[:n - 1], 0, [])
        assert O.rel_rms(m.forward(toks[n - 1], n - 1), want[n - 1]) < TOL["float32"], f"key at {far} (decoded)"
        # the prompt cut right behind the key, and two tokens before the end
        for cut in (far + 1, n - 2):
            if 0 < cut < n:
                m.forward_tokens(toks[:cut], 0, [])
                assert O.rel_rms(m.forward_tokens(toks[cut:], cut, [n - 1 - cut])[0], want[n - 1]) < TOL["float32"], f"key at {far}, cut at {cut}"
    m.close()


def one_key_attention(size, seed=7):
    """one parallel layer whose right mixer is switched off and whose convolutions look at the current token only; the query of
    token 49 and the key of token 48 share an unrotated dimension that no other token uses"""
    layer = P(heads=2, kv_heads=1, dim=8, vdim=8, conv=2, size=size, rot_dims=4, scale=1.0, softcap=40.0, left_scale=1.0, right_scale=0.0, mlp=None)
    cfg = O.make_config([layer], width=16, vocab=50, streams=2, residual_mult=1.0)
    W = O.random_weights(cfg, seed=seed)
    private_channel(W, [48, 49])
    for n in ("q", "k", "v"):
        W[f"l0.mix.left.{n}.conv"][:] = [0.0, 1.0]
        W[f"l0.mix.left.{n}.b"][:] = 0.0
    for name in ("l0.mix.left.q", "l0.mix.left.k"):
        W[name][:, 0] = 0.0
        W[name][5, 0] = 16.0   # after the whole-row norm this one dimension carries nearly all of q (in head 0) and of k
    W["l0.mix.left.q.norm"][:] = 1.0
    W["l0.mix.left.k.norm"][:] = 1.0
    return cfg, W


@pytest.mark.parametrize("window", [7, 64, 65, 100])
def test_keys_just_inside_and_just_outside_the_window(gpu_lib, tmp_path, window):
    cfg, W = one_key_attention(window)
    n = 200
    last = n - 1
    places = [last - window - 1, last - window, last - window + 1, last - window + 2, last - 1]
    check_one_key_matters(gpu_lib, tmp_path, cfg, W, n, places, 48, 49, seen=lambda p: last - p < window)


def test_a_far_key_is_found_among_hundreds(gpu_lib, tmp_path):
    cfg, W = one_key_attention(0, seed=8)
    n = 330
    check_one_key_matters(gpu_lib, tmp_path, cfg, W, n, [0, 1, 63, 64, 191, 192, n - 3], 48, 49, seen=lambda p: True)


def test_the_extra_softmax_entry_takes_weight_away(gpu_lib, tmp_path, monkeypatch):
    """the denominator holds one more term than there are keys.  A slow implementation without it answers very differently, and
    the library follows the one with it -- also across the key splits of a decode step"""
    cfg = O.make_config([P(size=0, right_scale=0.0, mlp=None)], streams=2)
    W = O.random_weights(cfg, seed=9)
    toks = tokens_for(cfg, 90, seed=1)
    want, _ = O.forward(cfg, W, toks)
    with monkeypatch.context() as mp:
        mp.setattr(O, "zero_sink_softmax", lambda s: np.exp(s - s.max()) / np.exp(s - s.max()).sum())
        assert O.rel_rms(O.forward(cfg, W, toks)[0], want) > 100 * TOL["float32"]
    m = open_model(gpu_lib, tmp_path, cfg, W, "float32")
    assert O.rel_rms(m.forward_tokens(toks, 0, list(range(90))), want) < TOL["float32"]
    for i in range(70, 90):
        m.forward_tokens(toks[:i], 0, [])
        assert O.rel_rms(m.forward(toks[i], i), want[i]) < TOL["float32"]
    m.close()


def test_the_delta_state_remembers_a_write_from_far_back(gpu_lib, tmp_path):
    """delta-rule layer with almost no decay: what token a wrote under a key direction that no other token uses is read back
    hundreds of tokens later by token b"""
    layer = D(heads=2, kv_heads=1, dim=8, vdim=8, conv=2, mlp=None)
    cfg = O.make_config([layer], width=16, vocab=50, streams=2, residual_mult=1.0)
    W = O.random_weights(cfg, seed=9)
    a_tok, b_tok, n = 48, 49, 300
    private_channel(W, [a_tok], 0)          # read by the key
    private_channel(W, [b_tok], 1)          # read by the query
    W["l0.mix.A_log"][:] = -9.0
    for name, dim in (("l0.mix.k", 0), ("l0.mix.q", 1)):
        W[name][:, dim] = 0.0
        W[name][3, :] = 0.0
        W[name][3, dim] = 4.0               # channel 3 is zero for every other token, and nearly the whole unit vector for this one
        W[name + ".conv"][3] = [0.0, 1.0]
    check_one_key_matters(gpu_lib, tmp_path, cfg, W, n, [0, 1, 7, 8, 150, n - 3], a_tok, b_tok, seen=lambda p: True)


def test_the_linear_attention_state_remembers_a_write_from_far_back(gpu_lib, tmp_path):
    """right mixer with decays close to one and the left mixer switched off"""
    layer = P(heads=2, kv_heads=1, dim=8, vdim=8, size=4, r_heads=2, r_dim=8, r_vdim=8, rank=2, left_scale=0.0, right_scale=1.0, mlp=None)
    cfg = O.make_config([layer], width=16, vocab=50, streams=2, residual_mult=1.0)
    W = O.random_weights(cfg, seed=10)
    a_tok, b_tok, n = 48, 49, 300
    private_channel(W, [a_tok], 0)
    private_channel(W, [b_tok], 1)
    W["l0.mix.right.a2.b"][:] = 12.0
    W["l0.mix.right.a2"] = O.bf16_round(W["l0.mix.right.a2"] * 0.1)
    for name, dim in (("l0.mix.right.k", 0), ("l0.mix.right.q", 1)):
        W[name][:, dim] = 0.0
        W[name][3, :] = 0.0
        W[name][3, dim] = 4.0
    check_one_key_matters(gpu_lib, tmp_path, cfg, W, n, [0, 1, 7, 8, 150, n - 3], a_tok, b_tok, seen=lambda p: True)


def test_cache_and_state_are_reused_by_the_next_sequence(gpu_lib, tmp_path):
    cfg = mixed_cfg()
    a, b = tokens_for(cfg, 90, seed=1), tokens_for(cfg, 33, seed=2)
    W = weights_for(cfg, a + b, seed=6)
    wa, _ = O.forward(cfg, W, a)
    wb, _ = O.forward(cfg, W, b)
    m = open_model(gpu_lib, tmp_path, cfg, W, "float32")
    assert O.rel_rms(m.forward_tokens(a, 0, [89]), wa[[89]]) < TOL["float32"]
    # a shorter sequence over the same positions: nothing of `a` (keys beyond position 32, its states, its convolution tails)
    # may show
    assert O.rel_rms(m.forward_tokens(b[:20], 0, [0, 19]), wb[[0, 19]]) < TOL["float32"]
    for i in range(20, 33):
        assert O.rel_rms(m.forward(b[i], i), wb[i]) < TOL["float32"]
    assert O.rel_rms(m.forward_tokens(a, 0, [0, 50]), wa[[0, 50]]) < TOL["float32"]
    # a new sequence that starts with single tokens (the first tokens of a sequence, decoded)
    for i in range(5):
        assert O.rel_rms(m.forward(b[i], i), wb[i]) < TOL["float32"]
    # the recurrent state stands at one position: a step elsewhere is refused, a restart is not
    with pytest.raises(gpu_lib.LmrsError, match="position"):
        m.forward_tokens(b[:3], 17, [])
    assert O.rel_rms(m.forward_tokens(b, 0, [32]), wb[[32]]) < TOL["float32"]
    m.close()


def test_first_tokens_and_a_prompt_of_one(gpu_lib, tmp_path):
    cfg = mixed_cfg()
    W = weights_for(cfg, [7, 7, 0, 1, 2], seed=8)
    m = open_model(gpu_lib, tmp_path, cfg, W, "float32")
    for toks in ([7], [7, 7], [0, 1, 2]):
        want, _ = O.forward(cfg, W, toks)
        assert O.rel_rms(m.forward_tokens(toks, 0, list(range(len(toks)))), want) < TOL["float32"]
        assert O.rel_rms(m.forward(toks[0], 0), want[0]) < TOL["float32"]
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_greedy_generation_through_the_generate_loop(gpu_lib, tmp_path, dtype):
    cfg = mixed_cfg(dtype)
    W = O.random_weights(cfg, seed=9)
    W["head"] = O.bf16_round(W["head"] * 6.0)   # clear winners
    prompt = tokens_for(cfg, 21, seed=4)
    n_new = 150   # decodes across two key-tile borders, through several key splits, and both windows pass over decoded tokens
    m = open_model(gpu_lib, tmp_path, cfg, W, dtype, max_tokens=21 + n_new)
    m.forward_tokens(prompt[:-1], 0, [])
    ids = m.generate_greedy(prompt[-1], len(prompt) - 1, n_new).tolist()
    assert len(ids) == n_new
    if dtype == "float32":
        # replay the produced sequence through the slow implementation: every pick must be its argmax or within a hair of it
        del O.CHOICE_GAPS[:]
        want, _ = O.forward(cfg, W, prompt + ids)
        if all(g > 1e-4 for g in O.CHOICE_GAPS):
            for i, t in enumerate(ids):
                row = want[len(prompt) - 1 + i]
                assert row[t] >= row.max() - 1e-3 * (row.max() - row.min()), f"generated token {i}"
    # forward_argmax is the same pick
    m.forward_tokens(prompt[:-1], 0, [])
    assert m.forward_argmax(prompt[-1], len(prompt) - 1) == ids[0]
    # decode steps replayed from CUDA graphs and launched one by one are the same arithmetic
    m.set_option("graphs", 0)
    m.forward_tokens(prompt[:-1], 0, [])
    assert m.generate_greedy(prompt[-1], len(prompt) - 1, n_new).tolist() == ids
    # ... and so are steps whose kernels are chained with programmatic dependent launch, replayed or not
    for graphs in (1, 0):
        m.set_option("graphs", graphs)
        m.set_option("pdl", 1)
        m.forward_tokens(prompt[:-1], 0, [])
        assert m.generate_greedy(prompt[-1], len(prompt) - 1, n_new).tolist() == ids
    with pytest.raises(gpu_lib.LmrsError):
        m.forward(1, 21 + n_new)   # beyond the cache
    m.close()


def test_tensor_core_products_equal_the_cuda_core_products(gpu_lib, tmp_path):
    """bf16 mode, shapes that are no multiples of the 128 x 128 x 64 tile, experts with very unequal loads: rows, outputs and
    K tails are masked or zero-filled, group borders fall inside tiles"""
    cfg = O.make_config([
        D(heads=5, kv_heads=1, dim=24, vdim=24, mlp=O.moe(experts=7, top=7, ff=72, shared=56)),
        P(heads=6, kv_heads=2, dim=32, vdim=20, size=50, rot_dims=16, r_heads=4, r_dim=16, r_vdim=24, rank=16, mlp=O.dense(ff=200)),
        D(heads=4, kv_heads=2, dim=40, vdim=40, mlp=O.moe(experts=9, top=9, ff=40, shared=0)),
        P(heads=4, kv_heads=4, dim=24, vdim=24, size=0, rot_dims=24, r_heads=3, r_dim=24, r_vdim=16, rank=8, mlp=O.moe(experts=3, top=3, ff=200, shared=24)),
    ], width=72, vocab=203)
    toks = tokens_for(cfg, 300)
    W = O.random_weights(cfg, seed=10)
    want, _ = O.forward(cfg, W, toks)
    m = open_model(gpu_lib, tmp_path, cfg, W, "bfloat16", max_tokens=320)
    a = m.forward_tokens(toks, 0, list(range(300)))
    m.set_option("tensor_cores", 0)
    b = m.forward_tokens(toks, 0, list(range(300)))
    assert typical_row_close(a, b, 5e-3) and not np.array_equal(a, b)   # different kernels, same numbers up to summation order
    assert typical_row_close(a, want, TOL["bfloat16"]) and typical_row_close(b, want, TOL["bfloat16"])
    m.close()


def test_grouped_experts_with_unequal_loads(gpu_lib, tmp_path):
    """real choices in float32: most tokens go to few experts, some experts get none"""
    cfg = O.make_config([D(mlp=O.moe(experts=11, top=2, ff=24, shared=16))], width=48)
    toks = tokens_for(cfg, 200, seed=3)
    W = weights_for(cfg, toks, seed=13)
    W["l0.mlp.router.b"][:] = O.bf16_round(np.linspace(3.0, -3.0, 11))
    if not O.clear_choices(cfg, W, toks, GAP):
        pytest.skip("a close routing decision")
    want, _ = O.forward(cfg, W, toks)
    m = open_model(gpu_lib, tmp_path, cfg, W, "float32")
    assert O.rel_rms(m.forward_tokens(toks, 0, list(range(200))), want) < TOL["float32"]
    m.close()


def test_configuration_errors_are_reported(gpu_lib, tmp_path):
    cfg = mixed_cfg()
    W = O.random_weights(cfg)
    W2 = {k: v for k, v in W.items() if k != "l3.mix.A_log"}
    with pytest.raises(gpu_lib.LmrsError, match="l3.mix.A_log"):
        gpu_lib.Transformer.open(O.write_model(str(tmp_path / "b"), cfg, W2))
    W3 = dict(W)
    W3["l1.mlp.e3.down"] = W["l1.mlp.e3.down"][:, :-1]
    with pytest.raises(gpu_lib.LmrsError, match="l1.mlp.e3.down"):
        gpu_lib.Transformer.open(O.write_model(str(tmp_path / "c"), cfg, W3))
    W4 = {k: v for k, v in W.items() if k != "l2.hc1.mix"}
    with pytest.raises(gpu_lib.LmrsError, match="l2.hc1.mix"):
        gpu_lib.Transformer.open(O.write_model(str(tmp_path / "e"), cfg, W4))
    bad = O.make_config([dict(D(), type="no_such_mixer")])
    with pytest.raises(gpu_lib.LmrsError, match="no_such_mixer"):
        gpu_lib.Transformer.open(O.write_model(str(tmp_path / "d"), bad, O.random_weights(O.make_config([D()]))))
    m = open_model(gpu_lib, tmp_path, cfg, W, "float32", max_tokens=16)
    with pytest.raises(gpu_lib.LmrsError):
        m.forward_tokens([1] * 17, 0, [])
    with pytest.raises(gpu_lib.LmrsError, match="token"):
        m.forward_tokens([cfg["vocab"]], 0, [])
    m.close()


def test_cached_rows_can_be_read_back(gpu_lib, tmp_path):
    cfg = O.make_config([D(mlp=None), P(mlp=None)])
    W = O.random_weights(cfg, seed=3)
    toks = tokens_for(cfg, 12)
    st = O.StepOracle(cfg, W)
    st.step(toks)
    m = open_model(gpu_lib, tmp_path, cfg, W, "float32")
    m.forward_tokens(toks, 0, [])
    k, v = m.read_kv(1, 0, 12, k_cols=2 * 12, v_cols=2 * 20)
    assert np.allclose(k.reshape(12, -1), st.state[1]["left"]["k"].reshape(12, -1), atol=1e-4)
    assert np.allclose(v.reshape(12, -1), st.state[1]["left"]["v"].reshape(12, -1), atol=1e-4)
    with pytest.raises(gpu_lib.LmrsError, match="state"):
        m.read_kv(0, 0, 12, k_cols=4, v_cols=4)
    m.close()


def test_the_command_line_generates_from_a_folder(gpu_lib, tmp_path):
    """lm.rs_b200/examples/generate on a model folder prints the ids that generate_greedy picks"""
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    subprocess.check_call(["make", "-C", os.path.join(root, "lm.rs_b200"), "-s", "examples"])
    cfg = mixed_cfg()
    W = O.random_weights(cfg, seed=11)
    d = O.write_model(str(tmp_path / "cli"), cfg, W)
    prompt = [3, 9, 27, 20]
    env = dict(os.environ, GENERATE_DTYPE="float32")
    r = subprocess.run([os.path.join(root, "lm.rs_b200", "examples", "generate"), d, "10"] + [str(t) for t in prompt],
                       capture_output=True, text=True, env=env)
    assert r.returncode == 0, r.stderr
    m = gpu_lib.Transformer.open(d, dtype="float32", max_tokens=32)
    m.forward_tokens(prompt[:-1], 0, [])
    assert [int(x) for x in r.stdout.split()] == m.generate_greedy(prompt[-1], 3, 10).tolist()
    m.close()


def test_trace_replay_writes_the_logits_asked_for(gpu_lib, tmp_path):
    """bin/trace_run: a prompt in portions, then single tokens, then a second request over the same cache and state"""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = mixed_cfg()
    a, b = tokens_for(cfg, 75, seed=5), tokens_for(cfg, 9, seed=6)
    W = weights_for(cfg, a + b, seed=12)
    d = O.write_model(str(tmp_path / "tr"), cfg, W)
    wa, _ = O.forward(cfg, W, a)
    wb, _ = O.forward(cfg, W, b)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": a[:66], "want": [0, 65]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": a[66:73], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": a[73:74], "want": [0]}], "end": []},
             {"step": 3, "entries": [{"id": "x", "tokens": a[74:75], "want": [0]}], "end": ["x"]},
             {"step": 4, "entries": [{"id": "y", "tokens": b, "want": [8, 2]}], "end": ["y"]}]
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "80"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done %d" % i for i in range(5)]
    assert not (out / "1.f32").exists()
    V = cfg["vocab"]
    for step, want in ((0, wa[[0, 65]]), (2, wa[[73]]), (3, wa[[74]]), (4, wb[[8, 2]])):
        got = np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(-1, V)
        assert O.rel_rms(got, want) < TOL["float32"], f"step {step}"
