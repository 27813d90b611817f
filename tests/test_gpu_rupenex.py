"""Rupenex folder models on the GPU against the slow float64 implementation of tests/rupenex_oracle.py.

Small random models (bf16-representable weights, so both operand modes load the same numbers) are written to a temporary
folder and opened through lmrs_b200.Transformer.open -- the entry point trace replay, forward, forward_argmax and
generate_greedy share.  float32 mode is held to 2e-4 of the logits' root mean square, bfloat16 mode to 4e-2.  For float32
the weights are drawn until no routing decision of the run is a close call.  In bfloat16 a run may legitimately take the
other expert where two scores are a hair apart (and a recurrent layer carries that on), so the bfloat16 comparisons against
the slow implementation use models whose routers choose all of their experts -- the weights still matter, no choice can
flip -- and the one bfloat16 test with real choices holds the typical row to the tolerance."""
import numpy as np
import pytest

import rupenex_oracle as O

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-4, "bfloat16": 4e-2}
GAP = 1e-4


def mixed_cfg(dtype="float32", **kw):
    """both mixers, both feed-forwards, a layer without one, grouped and ungrouped heads, windows shorter and longer than a key
    tile, sizes that are no powers of two and differ from each other; for bfloat16 every router chooses all of its outputs"""
    ff = (lambda e, i, t, f, s: O.moe(e, i, t, f, s)) if dtype == "float32" else (lambda e, i, t, f, s: O.moe(e, i, e + i, f, s))
    return O.make_config([
        O.ssm_layer(mlp=O.dense()),
        O.attention_layer(size=9, keep_first=3, mlp=ff(5, 2, 3, 24, 40)),
        O.ssm_layer(heads=2, vdim=20, state=20, groups=1, conv=2, norm_groups=1, mlp=ff(4, 0, 1, 16, 0)),
        O.attention_layer(heads=6, kv_heads=3, dim=8, vdim=12, size=70, keep_first=0, rot_dims=8, factor=None, mlp=None),
        O.attention_layer(heads=3, kv_heads=3, dim=16, vdim=8, size=0, rot_dims=6, mlp=O.dense(ff=30, limit=0.7)),
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
    assert m.args.model_type == gpu_lib.ModelType.RUPENEX and m.args.vocab_size == cfg["vocab"] and m.args.n_layers == 5
    m.set_option("keep_layers", 1)
    got = m.forward_tokens(toks, 0, list(range(85)))
    lo = m.layer_outputs(85)
    for li in range(5):   # the first layer that differs names the broken mechanism
        assert O.rel_rms(lo[li], outs[li]) < TOL[dtype], f"residual stream after layer {li}"
    assert O.rel_rms(got, want) < TOL[dtype]
    assert m.kernel_launches() > 0
    m.close()


# each mechanism alone: a one-layer model in which only that mechanism is not trivial, in shapes that take different branches
A, S = O.attention_layer, O.ssm_layer
ALONE = {
    "ssm": dict(layers=[S(mlp=None)]),
    "ssm_one_tap": dict(layers=[S(conv=1, mlp=None)]),
    "ssm_many_taps": dict(layers=[S(conv=7, mlp=None)]),
    "ssm_one_group_one_norm_part": dict(layers=[S(heads=3, groups=1, norm_groups=1, mlp=None)]),
    "ssm_a_group_per_head": dict(layers=[S(heads=3, groups=3, norm_groups=3, mlp=None)]),
    "ssm_norm_parts_across_heads": dict(layers=[S(heads=4, vdim=6, groups=2, norm_groups=3, mlp=None)]),
    "ssm_tiny_state": dict(layers=[S(heads=2, vdim=12, state=3, groups=1, mlp=None)]),
    "ssm_state_over_several_lanes": dict(layers=[S(heads=2, vdim=12, state=44, groups=1, mlp=None)]),
    "ssm_state_over_half_a_warp": dict(layers=[S(heads=2, vdim=12, state=72, groups=2, mlp=None)]),
    "ssm_state_over_a_warp": dict(layers=[S(heads=2, vdim=8, state=136, groups=2, mlp=None)]),
    "ssm_widest_state": dict(layers=[S(heads=1, vdim=6, state=264, groups=1, norm_groups=1, mlp=None)]),
    "ssm_wide_values": dict(layers=[S(heads=2, vdim=136, state=8, groups=2, mlp=None)]),
    "attention": dict(layers=[A(mlp=None)]),
    "attention_no_window": dict(layers=[A(size=0, mlp=None)]),
    "attention_window_of_one_with_kept_keys": dict(layers=[A(size=1, keep_first=2, mlp=None)]),
    "attention_nothing_kept": dict(layers=[A(size=5, keep_first=0, mlp=None)]),
    "attention_window_one_tile": dict(layers=[A(size=64, keep_first=1, mlp=None)]),
    "attention_window_tile_plus_one": dict(layers=[A(size=65, keep_first=5, mlp=None)]),
    "attention_kept_keys_over_a_tile_border": dict(layers=[A(size=3, keep_first=66, mlp=None)]),
    "attention_window_longer_than_the_prompt": dict(layers=[A(size=500, keep_first=7, mlp=None)]),
    "attention_no_rotation": dict(layers=[A(rot_dims=0, mlp=None)]),
    "attention_whole_head_rotated_unscaled": dict(layers=[A(rot_dims=12, factor=None, mlp=None)]),
    "attention_one_kv_head": dict(layers=[A(heads=5, kv_heads=1, size=33, mlp=None)]),
    "attention_ungrouped": dict(layers=[A(heads=3, kv_heads=3, dim=8, vdim=8, rot_dims=8, mlp=None)]),
    "attention_many_heads_per_kv_head": dict(layers=[A(heads=20, kv_heads=1, dim=8, vdim=8, rot_dims=4, mlp=None)]),
    "attention_wide_values": dict(layers=[A(heads=2, kv_heads=1, dim=8, vdim=72, size=40, rot_dims=2, mlp=None)]),
    "dense_ff": dict(layers=[A(size=500, mlp=O.dense())]),
    "dense_ff_that_clamps_hard": dict(layers=[A(size=500, mlp=O.dense(ff=33, limit=0.1))]),
    "experts": dict(layers=[A(size=500)]),
    "experts_top_one_no_identity_no_shared": dict(layers=[A(size=500, mlp=O.moe(experts=4, identity=0, top=1, shared=0))]),
    "experts_all_chosen": dict(layers=[A(size=500, mlp=O.moe(experts=3, identity=1, top=4))]),
    "experts_mostly_identity": dict(layers=[A(size=500, mlp=O.moe(experts=1, identity=5, top=2, ff=8, shared=8))]),
    "experts_many": dict(layers=[A(size=500, mlp=O.moe(experts=40, identity=3, top=5, ff=8, shared=16))]),
    "odd_width": dict(layers=[S(heads=3, vdim=6, state=10, groups=1, norm_groups=1), A(dim=10, vdim=6, rot_dims=6)], width=27, vocab=33),
    # rows too long for the norm kernels to hold in registers between their passes
    "very_wide_rows": dict(layers=[A(heads=2, kv_heads=1, dim=8, vdim=8, size=500, rot_dims=4, mlp=O.moe(experts=2, identity=1, top=2, ff=8, shared=8))],
                           width=4104, vocab=20),
    # one-row products whose output rows are few and long: the warps of a CTA split each row, the last CTA applies the norm
    "long_rows_into_a_narrow_stream": dict(layers=[A(heads=16, kv_heads=4, dim=16, vdim=64, size=500, rot_dims=16, mlp=O.dense(ff=1024)),
                                                   S(heads=16, vdim=64, state=16, groups=4, norm_groups=4, mlp=None)], width=64, vocab=40),
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


@pytest.mark.parametrize("state,vdim", [(44, 12), (72, 6), (100, 13), (128, 40)])
def test_scan_with_two_columns_per_thread(gpu_lib, tmp_path, state, vdim):
    """large models give every thread of the scan two adjacent columns of the state; forced here on small ones, with an odd
    number of columns too, for whole prompts, portions that continue the state, and single tokens"""
    cfg = O.make_config([S(heads=2, vdim=vdim, state=state, groups=1, norm_groups=1, mlp=None), S(heads=4, vdim=vdim, state=state, groups=2, conv=2, mlp=None)])
    toks = tokens_for(cfg, 50, seed=5)
    W = O.random_weights(cfg, seed=14, gain=2.0)
    want, _ = O.forward(cfg, W, toks)
    m = open_model(gpu_lib, tmp_path, cfg, W, "float32")
    one = m.forward_tokens(toks, 0, list(range(50)))
    m.set_option("ssm_cols", 2)
    two = m.forward_tokens(toks, 0, list(range(50)))
    assert O.rel_rms(two, want) < TOL["float32"] and np.array_equal(one, two)   # the same sums in the same order
    parts = np.concatenate([m.forward_tokens(toks[:9], 0, list(range(9))), m.forward_tokens(toks[9:11], 9, [0, 1])] +
                           [m.forward(toks[i], i).copy()[None] for i in range(11, 50)])
    assert O.rel_rms(parts, want) < TOL["float32"]
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
    """an input dimension becomes private to some tokens: their embedding is large there, every other token's is chosen so that
    the embedding's layer norm gives (nearly) zero there"""
    E = W["embed"]
    n = E.shape[1]
    E[:, dim] = np.delete(E, dim, 1).sum(1) / (n - 1)   # equals the row's mean: the norm takes it off
    E[toks, dim] = 8.0
    W["embed"] = O.bf16_round(E)
    W["embed.norm"][dim] = 1.0


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


def one_key_attention(size, keep_first, seed=7):
    """one attention layer in which the query of token 49 and the key of token 48 share an unrotated dimension that no other
    token uses"""
    layer = O.attention_layer(heads=2, kv_heads=1, dim=8, vdim=8, size=size, keep_first=keep_first, rot_dims=4, scale=1.0, mlp=None)
    cfg = O.make_config([layer], width=16, vocab=50, logit_scale=1.0)
    W = O.random_weights(cfg, seed=seed)
    private_channel(W, [48, 49])
    for name in ("l0.mix.q", "l0.mix.k"):
        W[name][:, 0] = 0.0
        W[name][5, 0] = 16.0   # after the head's norm this one dimension carries nearly all of q (head 0) and of k
    W["l0.mix.sink"][:] = 1.0
    W["l0.ls1"][:] = 1.0
    return cfg, W


@pytest.mark.parametrize("window", [7, 64, 65, 100])
def test_keys_just_inside_and_just_outside_the_window(gpu_lib, tmp_path, window):
    cfg, W = one_key_attention(window, 0)
    n = 200
    last = n - 1
    places = [last - window - 1, last - window, last - window + 1, last - window + 2, last - 1]
    check_one_key_matters(gpu_lib, tmp_path, cfg, W, n, places, 48, 49, seen=lambda p: last - p < window)


@pytest.mark.parametrize("window,keep", [(7, 3), (64, 1), (5, 64), (3, 70)])
def test_the_first_keys_stay_visible_and_the_next_ones_do_not(gpu_lib, tmp_path, window, keep):
    cfg, W = one_key_attention(window, keep)
    n = 200
    last = n - 1
    places = sorted({0, keep - 1, keep, keep + 1, last - window, last - window + 1})
    check_one_key_matters(gpu_lib, tmp_path, cfg, W, n, places, 48, 49, seen=lambda p: last - p < window or p < keep)


def test_a_far_key_is_found_among_hundreds(gpu_lib, tmp_path):
    cfg, W = one_key_attention(0, 0, seed=8)
    n = 330
    check_one_key_matters(gpu_lib, tmp_path, cfg, W, n, [0, 1, 63, 64, 191, 192, n - 3], 48, 49, seen=lambda p: True)


def test_a_large_sink_takes_the_weight_away(gpu_lib, tmp_path):
    """the sink is no key: it only enlarges the denominator.  With a sink far above every score the mixer's output all but
    vanishes; dropping the sink from the slow implementation moves the answer a lot, and the library follows the sink"""
    cfg, W = one_key_attention(0, 0, seed=9)
    toks = tokens_for(cfg, 90, seed=1)
    W["l0.mix.sink"][:] = [6.0, -3.0]
    want, _ = O.forward(cfg, W, toks)
    Wn = {k: v for k, v in W.items() if k != "l0.mix.sink"}
    assert O.rel_rms(O.forward(cfg, Wn, toks)[0], want) > 100 * TOL["float32"]
    m = open_model(gpu_lib, tmp_path, cfg, W, "float32")
    assert O.rel_rms(m.forward_tokens(toks, 0, list(range(90))), want) < TOL["float32"]
    for i in range(70, 90):   # decoded: the sink belongs to one of the key splits only
        m.forward_tokens(toks[:i], 0, [])
        assert O.rel_rms(m.forward(toks[i], i), want[i]) < TOL["float32"]
    m.close()


def test_the_state_remembers_a_write_from_far_back(gpu_lib, tmp_path):
    """state-space layer with almost no decay: what token a wrote into a state row that no other token writes is read back
    hundreds of tokens later by token b"""
    layer = O.ssm_layer(heads=2, vdim=8, state=8, groups=1, conv=2, norm_groups=1, mlp=None)
    cfg = O.make_config([layer], width=16, vocab=50, logit_scale=1.0)
    W = O.random_weights(cfg, seed=9)
    a_tok, b_tok, n = 48, 49, 300
    private_channel(W, [a_tok], 0)          # read by the write side (B)
    private_channel(W, [b_tok], 1)          # read by the read side (C)
    W["l0.mix.A_log"][:] = -9.0
    inner = 16
    for row, dim in ((2 * inner + 3, 0), (2 * inner + 8 + 3, 1)):   # B row 3 and C row 3 of the only group
        W["l0.mix.in"][:, dim] = 0.0
        W["l0.mix.in"][row, :] = 0.0
        W["l0.mix.in"][row, dim] = 4.0
        ch = row - inner
        W["l0.mix.conv"][ch] = [0.0, 1.0]   # the channel looks at the current token only
        W["l0.mix.conv.b"][ch] = -2.0       # ... and is nearly shut for every other token
    W["l0.ls1"][:] = 1.0
    check_one_key_matters(gpu_lib, tmp_path, cfg, W, n, [0, 1, 7, 8, 150, n - 3], a_tok, b_tok, seen=lambda p: True)


def test_cache_and_state_are_reused_by_the_next_sequence(gpu_lib, tmp_path):
    cfg = mixed_cfg()
    a, b = tokens_for(cfg, 90, seed=1), tokens_for(cfg, 33, seed=2)
    W = weights_for(cfg, a + b, seed=6)
    wa, _ = O.forward(cfg, W, a)
    wb, _ = O.forward(cfg, W, b)
    m = open_model(gpu_lib, tmp_path, cfg, W, "float32")
    assert O.rel_rms(m.forward_tokens(a, 0, [89]), wa[[89]]) < TOL["float32"]
    # a shorter sequence over the same positions: nothing of `a` (keys beyond position 32, its state, its convolution tail)
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
    cfg = mixed_cfg(dtype, logit_scale=3.0)
    W = O.random_weights(cfg, seed=9)
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
        O.ssm_layer(heads=5, vdim=24, state=40, groups=1, norm_groups=5, mlp=O.moe(experts=7, identity=2, top=2, ff=72, shared=56)),
        O.attention_layer(heads=6, kv_heads=2, dim=32, vdim=20, size=50, keep_first=4, rot_dims=16, mlp=O.dense(ff=200)),
        O.ssm_layer(heads=4, vdim=40, state=24, groups=2, mlp=O.moe(experts=9, identity=0, top=4, ff=40, shared=0)),
        O.attention_layer(heads=4, kv_heads=4, dim=24, vdim=24, size=0, rot_dims=24, mlp=O.moe(experts=3, identity=1, top=1, ff=200, shared=24)),
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


def test_configuration_errors_are_reported(gpu_lib, tmp_path):
    cfg = mixed_cfg()
    W = O.random_weights(cfg)
    W2 = {k: v for k, v in W.items() if k != "l2.mix.A_log"}
    with pytest.raises(gpu_lib.LmrsError, match="l2.mix.A_log"):
        gpu_lib.Transformer.open(O.write_model(str(tmp_path / "b"), cfg, W2))
    W3 = dict(W)
    W3["l1.mlp.e3.down"] = W["l1.mlp.e3.down"][:, :-1]
    with pytest.raises(gpu_lib.LmrsError, match="l1.mlp.e3.down"):
        gpu_lib.Transformer.open(O.write_model(str(tmp_path / "c"), cfg, W3))
    bad = O.make_config([dict(O.attention_layer(), type="no_such_mixer")])
    with pytest.raises(gpu_lib.LmrsError, match="no_such_mixer"):
        gpu_lib.Transformer.open(O.write_model(str(tmp_path / "d"), bad, O.random_weights(O.make_config([O.attention_layer()]))))
    m = open_model(gpu_lib, tmp_path, cfg, W, "float32", max_tokens=16)
    with pytest.raises(gpu_lib.LmrsError):
        m.forward_tokens([1] * 17, 0, [])
    with pytest.raises(gpu_lib.LmrsError, match="token"):
        m.forward_tokens([cfg["vocab"]], 0, [])
    m.close()


def test_cached_rows_can_be_read_back(gpu_lib, tmp_path):
    cfg = O.make_config([O.ssm_layer(mlp=None), O.attention_layer(mlp=None)])
    W = O.random_weights(cfg, seed=3)
    toks = tokens_for(cfg, 12)
    st = O.StepOracle(cfg, W)
    st.step(toks)
    m = open_model(gpu_lib, tmp_path, cfg, W, "float32")
    m.forward_tokens(toks, 0, [])
    k, v = m.read_kv(1, 0, 12, k_cols=2 * 12, v_cols=2 * 20)
    assert np.allclose(k.reshape(12, -1), st.state[1]["k"].reshape(12, -1), atol=1e-4)
    assert np.allclose(v.reshape(12, -1), st.state[1]["v"].reshape(12, -1), atol=1e-4)
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
