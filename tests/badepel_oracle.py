"""Plain, slow float64 implementation of the Badepel architecture: test infrastructure only.

One function per mechanism, written from the equations below in numpy; it shares no code with the library.

    rms(v)         v / sqrt(mean(v^2) + eps)
    streams        the residual is S copies X[0..S) of the embedding row.  Sublayer q of a layer (1 mixer, 2 feed-forward) with
                   vectors a = hcq.in [S], b = hcq.out [S] and matrix M = hcq.mix [S, S] (row = source, column = target):
                     u = sum_s a[s] X[s];   y = sublayer(rms(u) * norm_q);   X'[t] = sum_s M[s, t] X[s] + m b[t] y
                   with m = residual_mult; a model without the hc tensors has S = 1, a = b = M = 1.  The layer's output and
                   the final norm's input is sum_s X[s].
    mixer P        'parallel': two mixers read the same input, result = left_scale * L + right_scale * R
      L            grouped-head attention: q, k, v = W h + bias; a short causal convolution over time on every channel of
                   q, k, v (no activation); q and k each RMS-normed over their WHOLE row (all heads at once) with a weight;
                   the first rot.dims dimensions of every q and k head turned in neighbouring pairs (2i, 2i+1) by
                   position * base^(-2i/dims); s = scale q.k; s <- cap tanh(s / cap); i sees j when 0 <= i - j < mask.size;
                   p_j = exp(s_j) / (1 + sum exp(s)); W_o on the joined heads
      R            gated linear attention: q = W_q h / sqrt(dim), k = W_k h, v = W_v h; a = sigmoid(W_a2 W_a1 h + bias)^(1/tau)
                   per head and key channel; S <- diag(a) S + k v^T; o = S^T q; o <- rms(o) * w per head; joined heads times
                   silu(W_g h); W_o
    mixer D        'delta': q, k (kv_heads x dim), v (heads x vdim) = W h; causal convolution, then silu; q, k to unit length
                   per head (x / sqrt(sum x^2 + 1e-6)), q also / sqrt(dim); beta = sigmoid(W_b h);
                   g = exp(-exp(A_log) softplus(W_a h + dt_bias)) per head; S <- g S; u = beta (v - S^T k); S <- S + k u^T;
                   o = S^T q; o <- rms(o) * w per head, times silu(W_g h); W_o
    ff dense       W_down (silu(W_gate h) * (W_up h))
    ff routed      z = W_r h + b_r; the `top` largest z are chosen, weights = softmax over the chosen z; an expert is
                   g = min(W_gate h, limit), u = clip(W_up h, -limit, limit), W_down (g sigmoid(1.702 g) (u + 1)); a shared
                   expert of the same form (own size and limit) is added for every token
    logits         W_head (rms(sum_s X[s]) * w_final)

StepOracle carries the state (recurrent matrices, convolution tails, key/value lists) from call to call, so the
whole-sequence functions and the incremental form check each other.  make_config / random_weights / write_model build
small random model folders (config.json + model.safetensors with bf16 tensors).
"""
import json
import math
import os
import struct

import numpy as np


# ---- number formats -----------------------------------------------------------------------------------------------------
def to_bf16_bits(a):
    u = np.asarray(a, np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_round(a):
    return (to_bf16_bits(a).astype(np.uint32) << 16).view(np.float32).astype(np.float64)


# ---- small functions --------------------------------------------------------------------------------------------------------
def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


# ---- residual streams -------------------------------------------------------------------------------------------------------
def streams_read(X, a):
    """X [T, S, width], a [S] -> the sublayer's input before its norm, [T, width]"""
    return np.einsum("s,tsw->tw", a, X)


def streams_write(X, y, M, b, m):
    """every stream from the old ones at once: X'[:, t] = sum_s M[s, t] X[:, s] + m b[t] y"""
    return np.einsum("su,tsw->tuw", M, X) + m * b[None, :, None] * y[:, None, :]


def stream_weights(W, name, S):
    """(in, out, mix) of one sublayer; a model without these tensors has one stream that is read and written as it is"""
    if name + ".in" in W:
        return W[name + ".in"], W[name + ".out"], W[name + ".mix"]
    assert S == 1
    return np.ones(1), np.ones(1), np.ones((1, 1))


# ---- short causal convolution -----------------------------------------------------------------------------------------------
def causal_conv(u, w, tail):
    """u [T, C]; w [C, taps], last column on the current token; tail [taps-1, C]: the inputs before u (zeros at a start).
    -> (y [T, C], new tail)"""
    taps = w.shape[1]
    ext = np.concatenate([tail, u], 0)
    y = np.zeros_like(u)
    for j in range(taps):
        y += w[:, j] * ext[j:j + u.shape[0]]
    return y, ext[ext.shape[0] - (taps - 1):]


# ---- mixer P, left: windowed attention with a zero sink ------------------------------------------------------------------------
def rotate_pairs(x, positions, rot):
    """x [T, heads, n >= dims]: dimensions 2i and 2i+1 (i < dims/2) turn together by positions * base^(-2i/dims)"""
    if not rot or not rot.get("dims"):
        return x
    d = rot["dims"]
    f = np.array([rot["base"] ** (-2.0 * i / d) for i in range(d // 2)], np.float64)
    ang = np.asarray(positions, np.float64)[:, None, None] * f[None, None, :]
    c, s = np.cos(ang), np.sin(ang)
    out = x.copy()
    u, v = x[..., 0:d:2], x[..., 1:d:2]
    out[..., 0:d:2] = u * c - v * s
    out[..., 1:d:2] = v * c + u * s
    return out


def in_window(i, j, mask):
    """may position i look at position j?"""
    if j > i:
        return False
    return not mask or not mask.get("size") or i - j < mask["size"]


def soft_cap(s, cap):
    return cap * np.tanh(s / cap) if cap else s


def zero_sink_softmax(s):
    """exp(s_j) / (1 + sum exp(s)): a further entry of score 0 that carries no value"""
    mx = max(float(np.max(s)), 0.0)
    e = np.exp(s - mx)
    return e / (math.exp(-mx) + np.sum(e))


def window_mixer(h, W, p, m, eps, state, pos0):
    """state: 'tail' of the convolution, 'k' [n, G, dk] turned keys and 'v' [n, G, dv] of the positions before pos0"""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(pos0, pos0 + T)
    u = np.concatenate([h @ W[p + n].T + W[p + n + ".b"] for n in ("q", "k", "v")], 1)
    taps = m.get("conv", 0)
    if taps:
        w = np.concatenate([W[p + n + ".conv"] for n in ("q", "k", "v")], 0)
        u, state["tail"] = causal_conv(u, w, state.get("tail", np.zeros((taps - 1, u.shape[1]))))
    q, k, v = u[:, :H * dk], u[:, H * dk:(H + G) * dk], u[:, (H + G) * dk:]
    q = rotate_pairs((rms(q, eps) * W[p + "q.norm"]).reshape(T, H, dk), pos, m.get("rot"))
    k = rotate_pairs((rms(k, eps) * W[p + "k.norm"]).reshape(T, G, dk), pos, m.get("rot"))
    v = v.reshape(T, G, dv)
    keys = np.concatenate([state["k"], k], 0) if "k" in state else k
    vals = np.concatenate([state["v"], v], 0) if "v" in state else v
    state["k"], state["v"] = keys, vals
    out = np.zeros((T, H, dv))
    for t in range(T):
        i = pos0 + t
        js = [j for j in range(i + 1) if in_window(i, j, m.get("mask"))]
        for hh in range(H):
            g = hh // (H // G)
            s = soft_cap(keys[js, g] @ q[t, hh] * m["scale"], m.get("softcap"))
            out[t, hh] = zero_sink_softmax(s) @ vals[js, g]
    return out.reshape(T, H * dv) @ W[p + "o"].T


# ---- mixer P, right: gated linear attention -------------------------------------------------------------------------------------
def gla_scan(q, k, v, a, S):
    """q, k, a [T, H, dk], v [T, H, dv], S [H, dk, dv] (updated in place) -> o [T, H, dv]"""
    o = np.zeros(v.shape)
    for t in range(q.shape[0]):
        for hh in range(q.shape[1]):
            S[hh] = a[t, hh][:, None] * S[hh] + np.outer(k[t, hh], v[t, hh])
            o[t, hh] = S[hh].T @ q[t, hh]
    return o


def gla_mixer(h, W, p, m, eps, state):
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).reshape(T, H, dk) / math.sqrt(dk)
    k = (h @ W[p + "k"].T).reshape(T, H, dk)
    v = (h @ W[p + "v"].T).reshape(T, H, dv)
    z = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "a2.b"]
    a = np.exp(-softplus(-z) / m["tau"]).reshape(T, H, dk)       # sigmoid(z)^(1/tau)
    if "S" not in state:
        state["S"] = np.zeros((H, dk, dv))
    o = rms(gla_scan(q, k, v, a, state["S"]), eps) * W[p + "norm"]
    return (o.reshape(T, H * dv) * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


def parallel_mixer(h, W, p, m, eps, state, pos0):
    left = window_mixer(h, W, p + "left.", m["left"], eps, state.setdefault("left", {}), pos0)
    right = gla_mixer(h, W, p + "right.", m["right"], eps, state.setdefault("right", {}))
    return m["left_scale"] * left + m["right_scale"] * right


# ---- mixer D: gated delta rule ----------------------------------------------------------------------------------------------------
def unit(x):
    return x / np.sqrt(np.sum(x * x, axis=-1, keepdims=True) + 1e-6)


def delta_scan(q, k, v, g, beta, S):
    """q, k [T, H, dk] (already per value head), v [T, H, dv], g, beta [T, H], S [H, dk, dv] (updated in place)"""
    o = np.zeros(v.shape)
    for t in range(q.shape[0]):
        for hh in range(q.shape[1]):
            S[hh] *= g[t, hh]
            u = beta[t, hh] * (v[t, hh] - S[hh].T @ k[t, hh])
            S[hh] += np.outer(k[t, hh], u)
            o[t, hh] = S[hh].T @ q[t, hh]
    return o


def delta_mixer(h, W, p, m, eps, state):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    u = np.concatenate([h @ W[p + n].T for n in ("q", "k", "v")], 1)
    w = np.concatenate([W[p + n + ".conv"] for n in ("q", "k", "v")], 0)
    u, state["tail"] = causal_conv(u, w, state.get("tail", np.zeros((m["conv"] - 1, u.shape[1]))))
    u = silu(u)
    q = unit(u[:, :G * dk].reshape(T, G, dk)) / math.sqrt(dk)
    k = unit(u[:, G * dk:2 * G * dk].reshape(T, G, dk))
    v = u[:, 2 * G * dk:].reshape(T, H, dv)
    rep = H // G
    q, k = np.repeat(q, rep, axis=1), np.repeat(k, rep, axis=1)      # value head hh reads q/k head hh // rep
    beta = sigmoid(h @ W[p + "b"].T)
    g = np.exp(-np.exp(W[p + "A_log"]) * softplus(h @ W[p + "a"].T + W[p + "dt_bias"]))
    if "S" not in state:
        state["S"] = np.zeros((H, dk, dv))
    o = rms(delta_scan(q, k, v, g, beta, state["S"]), eps) * W[p + "norm"]
    return (o.reshape(T, H * dv) * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


# ---- feed-forward ---------------------------------------------------------------------------------------------------------------------
def dense_ff(h, W, p):
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


CHOICE_GAPS = []   # of every routing decision made: lowest chosen logit minus highest rejected one


def route(h, W, p, r):
    """-> (chosen experts [T, top], weights [T, top]): the largest logits, softmax over the chosen ones only"""
    z = h @ W[p + "router"].T + W[p + "router.b"]
    idx = np.argsort(-z, axis=1, kind="stable")[:, :r["top"]]
    zc = np.take_along_axis(z, idx, 1)
    if r["top"] < z.shape[1]:
        rest = np.sort(z, axis=1)[:, ::-1][:, r["top"]]
        CHOICE_GAPS.extend((zc.min(1) - rest).tolist())
    e = np.exp(zc - zc.max(1, keepdims=True))
    return idx, e / e.sum(1, keepdims=True)


def expert(h, W, p, limit):
    g = np.minimum(h @ W[p + "gate"].T, limit)
    u = np.clip(h @ W[p + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def routed_ff(h, W, p, f):
    idx, wts = route(h, W, p, f["router"])
    limit = f["expert"].get("limit", math.inf)
    y = np.zeros((h.shape[0], W[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, w in zip(idx[t], wts[t]):
            y[t] += w * expert(h[t:t + 1], W, f"{p}e{e}.", limit)[0]
    if f.get("shared"):
        y += expert(h, W, p + "shared.", f["shared"].get("limit", math.inf))
    return y


# ---- the model -----------------------------------------------------------------------------------------------------------------------------
class StepOracle:
    """Feeds tokens in portions; keeps every layer's state between calls."""

    def __init__(self, cfg, W):
        self.cfg, self.W = cfg, {k: np.asarray(v, np.float64) for k, v in W.items()}
        self.state = [dict() for _ in cfg["layers"]]
        self.pos = 0

    def step(self, tokens):
        """-> (logits [T, vocab], sum of the residual streams after every layer [layers, T, width])"""
        cfg, W, eps = self.cfg, self.W, self.cfg["norm"]["eps"]
        S, m = cfg.get("streams", 1), cfg.get("residual_mult", 1.0)
        X = np.repeat(W["embed"][np.asarray(tokens, np.int64)][:, None, :], S, axis=1)
        outs = []
        for i, L in enumerate(cfg["layers"]):
            p = f"l{i}."
            a, b, M = stream_weights(W, p + "hc1", S)
            h = rms(streams_read(X, a), eps) * W[p + "norm1"]
            if L["type"] == "parallel":
                y = parallel_mixer(h, W, p + "mix.", L["mixer"], eps, self.state[i], self.pos)
            elif L["type"] == "delta":
                y = delta_mixer(h, W, p + "mix.", L["mixer"], eps, self.state[i])
            else:
                raise ValueError(L["type"])
            X = streams_write(X, y, M, b, m)
            f = L.get("mlp")
            if f:
                a, b, M = stream_weights(W, p + "hc2", S)
                h = rms(streams_read(X, a), eps) * W[p + "norm2"]
                y = dense_ff(h, W, p + "mlp.") if f.get("kind", "dense") == "dense" else routed_ff(h, W, p + "mlp.", f)
                X = streams_write(X, y, M, b, m)
            outs.append(X.sum(1))
        self.pos += len(tokens)
        logits = (rms(X.sum(1), eps) * W["final.norm"]) @ W["head"].T
        return logits, np.stack(outs)


def forward(cfg, W, tokens):
    return StepOracle(cfg, W).step(tokens)


def clear_choices(cfg, W, tokens, gap):
    """True when no routing decision of this run is closer than `gap` (a test in reduced precision must not rest on one)"""
    del CHOICE_GAPS[:]
    forward(cfg, W, tokens)
    return all(g > gap for g in CHOICE_GAPS)


def rel_rms(got, want):
    """root mean square of the difference over that of `want`, means over the last axis taken off"""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return float(np.sqrt(np.mean(d * d)) / (np.sqrt(np.mean(w * w)) + 1e-30))


# ---- small random models -----------------------------------------------------------------------------------------------------------------
def dense(ff=56):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, top=2, ff=24, limit=1.25, shared=40, shared_limit=2.5):
    f = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared:
        f["shared"] = {"ff": shared, "limit": shared_limit}
    return f


def parallel_layer(heads=4, kv_heads=2, dim=12, vdim=20, conv=3, size=9, rot_dims=8, base=100.0, scale=0.4, softcap=8.0,
                   r_heads=3, r_dim=8, r_vdim=12, tau=4.0, rank=5, left_scale=1.3, right_scale=0.8, mlp="default"):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "scale": scale, "softcap": softcap}
    if size:
        left["mask"] = {"size": size}
    if rot_dims:
        left["rot"] = {"base": base, "dims": rot_dims}
    right = {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "tau": tau, "rank": rank}
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": moe() if mlp == "default" else mlp}


def delta_layer(heads=4, kv_heads=2, dim=12, vdim=10, conv=4, mlp="default"):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": dense() if mlp == "default" else mlp}


def make_config(layers, width=40, vocab=70, eps=1e-5, streams=3, residual_mult=0.6):
    """the low rank of the decay projection ('rank' of a right mixer) is not a configuration entry of the design: it is the
    shape of a1.  It rides in the dictionary for tensor_table and is dropped from the written config.json."""
    return {"architecture": "Badepel", "width": width, "vocab": vocab, "norm": {"eps": eps}, "streams": streams,
            "residual_mult": residual_mult, "layers": layers}


def tensor_table(cfg, hc=True):
    """[(name, shape, kind)]; kind: matrix | table | gain | shift | conv | rate | read | write | mixing"""
    w, S = cfg["width"], cfg.get("streams", 1)
    out = [("embed", (cfg["vocab"], w), "table")]
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        q = p + "mix."
        out += [(p + "norm1", (w,), "gain")]
        if L["type"] == "parallel":
            l, r = m["left"], m["right"]
            H, G, dk, dv = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
            ql = q + "left."
            for n, rows in (("q", H * dk), ("k", G * dk), ("v", G * dv)):
                out += [(ql + n, (rows, w), "matrix"), (ql + n + ".b", (rows,), "shift")]
                if l.get("conv"):
                    out.append((ql + n + ".conv", (rows, l["conv"]), "conv"))
            out += [(ql + "q.norm", (H * dk,), "gain"), (ql + "k.norm", (G * dk,), "gain"), (ql + "o", (w, H * dv), "matrix")]
            Hr, dkr, dvr, ra = r["heads"], r["dim"], r["vdim"], r.get("rank", 4)
            qr = q + "right."
            out += [(qr + "q", (Hr * dkr, w), "matrix"), (qr + "k", (Hr * dkr, w), "matrix"), (qr + "v", (Hr * dvr, w), "matrix"),
                    (qr + "g", (Hr * dvr, w), "matrix"), (qr + "o", (w, Hr * dvr), "matrix"), (qr + "norm", (dvr,), "gain"),
                    (qr + "a1", (ra, w), "matrix"), (qr + "a2", (Hr * dkr, ra), "matrix"), (qr + "a2.b", (Hr * dkr,), "decay")]
        else:
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for n, rows in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                out += [(q + n, (rows, w), "matrix"), (q + n + ".conv", (rows, m["conv"]), "conv")]
            out += [(q + "b", (H, w), "matrix"), (q + "A_log", (H,), "rate"), (q + "norm", (dv,), "gain"), (q + "a", (H, w), "matrix"),
                    (q + "dt_bias", (H,), "shift"), (q + "g", (H * dv, w), "matrix"), (q + "o", (w, H * dv), "matrix")]
        f = L.get("mlp")
        if f:
            out += [(p + "norm2", (w,), "gain")]
            if f.get("kind", "dense") == "dense":
                out += [(p + "mlp.gate", (f["ff"], w), "matrix"), (p + "mlp.up", (f["ff"], w), "matrix"), (p + "mlp.down", (w, f["ff"]), "matrix")]
            else:
                r = f["router"]
                for e in range(r["experts"]):
                    ff = f["expert"]["ff"]
                    out += [(f"{p}mlp.e{e}.gate", (ff, w), "matrix"), (f"{p}mlp.e{e}.up", (ff, w), "matrix"), (f"{p}mlp.e{e}.down", (w, ff), "matrix")]
                out += [(p + "mlp.router", (r["experts"], w), "matrix"), (p + "mlp.router.b", (r["experts"],), "shift")]
                if f.get("shared"):
                    ff = f["shared"]["ff"]
                    out += [(p + "mlp.shared.gate", (ff, w), "matrix"), (p + "mlp.shared.up", (ff, w), "matrix"), (p + "mlp.shared.down", (w, ff), "matrix")]
        if hc:
            for s in ("hc1", "hc2") if f else ("hc1",):
                out += [(f"{p}{s}.in", (S,), "read"), (f"{p}{s}.out", (S,), "write"), (f"{p}{s}.mix", (S, S), "mixing")]
    return out + [("final.norm", (w,), "gain"), ("head", (cfg["vocab"], w), "matrix")]


def random_weights(cfg, seed=0, gain=1.0, hc=True):
    """bf16-representable float64 weights"""
    rng = np.random.default_rng(seed)
    W = {}
    for name, shape, kind in tensor_table(cfg, hc):
        n = int(np.prod(shape)) if shape else 1
        if kind == "matrix":
            a = rng.standard_normal(n) * gain / math.sqrt(shape[-1])
            if name.endswith("router"):
                a *= 3.0
        elif kind == "table":
            a = rng.standard_normal(n)
        elif kind == "gain":
            a = 1.0 + 0.2 * rng.standard_normal(n)
        elif kind == "shift":
            a = 0.3 * rng.standard_normal(n)
        elif kind == "conv":
            a = rng.standard_normal(n) * 0.6
        elif kind == "rate":
            a = -1.0 + rng.standard_normal(n)
        elif kind == "decay":
            a = 2.0 + rng.standard_normal(n)
        elif kind == "read":
            a = 1.0 / shape[0] + 0.2 * rng.standard_normal(n)
        elif kind == "write":
            a = 1.0 + 0.3 * rng.standard_normal(n)
        elif kind == "mixing":
            a = (np.eye(shape[0]) + 0.15 * rng.standard_normal(shape)).reshape(-1)
        else:
            raise ValueError(kind)
        W[name] = bf16_round(a).reshape(shape)
    return W


def written_config(cfg):
    """config.json as the library reads it: without the entries that only tensor_table uses"""
    c = json.loads(json.dumps(cfg))
    for L in c["layers"]:
        if L["type"] == "parallel":
            L["mixer"]["right"].pop("rank", None)
    return c


def write_model(folder, cfg, W):
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(written_config(cfg), f)
    header, blobs, off = {}, [], 0
    for name, a in W.items():
        b = to_bf16_bits(np.asarray(a, np.float32)).tobytes()
        header[name] = {"dtype": "BF16", "shape": list(np.shape(a)), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj)
        for b in blobs:
            f.write(b)
    return folder
