"""Plain, slow float64 implementation of the Rupenex architecture: test infrastructure only.

One function per mechanism, written from the equations below in numpy; it shares no code with the library.

    embedding      x = LN(embed[token]) * w_embed_norm
    layer          x <- x + ls1 * LN1(mixer(x));  x <- x + ls2 * LN2(ff(x))     (the sublayers read x itself; the second line
                   only with a feed-forward);  LN(v) = (v - mean) / sqrt(var + eps) * w, no bias
    rms(v)         v / sqrt(mean(v^2) + eps)
    mixer A        attention (attention_*): grouped heads; q, k <- rms per head * w (one weight vector for all heads);
                     rotation of dimension pairs (i, i + dims/2) of the first `dims` dimensions by position * base^(-2i/dims)
                     / factor;  s = scale * q.k;  i sees j <= i when i - j < size or j < keep_first;  softmax whose
                     denominator also holds exp(sink_head);  heads * sigmoid(W_g h);  W_o
    mixer M        state-space recurrence (ssm_*): [z | x | B | C | dt] = W_in h;  (x, B, C) <- silu(causal_conv + bias);
                     dt <- softplus(dt + dt_bias);  S <- exp(-exp(A_log) dt) S + dt B x^T;  y = S^T C + D x;
                     y <- y * silu(z), rms in norm_groups equal parts, * w;  W_o
    ff dense       g = min(W_gate h, limit);  u = clip(W_up h, -limit, limit);  W_down (g sigmoid(1.702 g) (u + 1))
    ff routed      s = softmax(W_r h) over experts + identity experts;  the `top` largest of s + correction are chosen;
                     weights = s_chosen / (sum s_chosen + 1e-20);  expert(h) = W_down relu(W_up h)^2;  an identity expert
                     returns h;  a shared expert of the same form is added for every token
    logits         logit_scale * W_head (LN(x) * w_final)

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
def layer_norm(x, w, eps):
    mu = np.mean(x, axis=-1, keepdims=True)
    d = x - mu
    return d / np.sqrt(np.mean(d * d, axis=-1, keepdims=True) + eps) * w


def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


# ---- mixer A: attention ---------------------------------------------------------------------------------------------------------
def rot_freqs(rot):
    d = rot["dims"]
    factor = (rot.get("scaling") or {}).get("factor", 1.0)
    return np.array([rot["base"] ** (-2.0 * i / d) / factor for i in range(d // 2)], np.float64)


def rotate_halves(x, positions, rot):
    """x [T, heads, n >= dims]: dimension i < dims/2 and dimension i + dims/2 turn together by positions * f_i"""
    if not rot or not rot.get("dims"):
        return x
    d = rot["dims"]
    half = d // 2
    ang = np.asarray(positions, np.float64)[:, None, None] * rot_freqs(rot)[None, None, :]
    c, s = np.cos(ang), np.sin(ang)
    out = x.copy()
    u, v = x[..., :half], x[..., half:d]
    out[..., :half] = u * c - v * s
    out[..., half:d] = v * c + u * s
    return out


def visible(i, j, mask):
    """may position i look at position j?"""
    if j > i:
        return False
    if not mask or not mask.get("size"):
        return True
    return i - j < mask["size"] or j < mask.get("keep_first", 0)


def sink_softmax(s, sink):
    """weights of the scores s [n] when the denominator also counts exp(sink) (sink None: an ordinary softmax)"""
    mx = np.max(s) if sink is None else max(np.max(s), sink)
    e = np.exp(s - mx)
    return e / (np.sum(e) + (0.0 if sink is None else math.exp(sink - mx)))


def attention_mixer(h, W, p, m, eps, state, pos0):
    """state: 'k' [n, G, dk] rotated keys and 'v' [n, G, dv] of the positions before pos0"""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(pos0, pos0 + T)
    q = (h @ W[p + "q"].T).reshape(T, H, dk)
    k = (h @ W[p + "k"].T).reshape(T, G, dk)
    v = (h @ W[p + "v"].T).reshape(T, G, dv)
    q = rotate_halves(rms(q, eps) * W[p + "q.norm"], pos, m.get("rot"))
    k = rotate_halves(rms(k, eps) * W[p + "k.norm"], pos, m.get("rot"))
    keys = np.concatenate([state["k"], k], 0) if "k" in state else k
    vals = np.concatenate([state["v"], v], 0) if "v" in state else v
    state["k"], state["v"] = keys, vals
    sink = W.get(p + "sink")
    out = np.zeros((T, H, dv))
    for t in range(T):
        i = pos0 + t
        js = [j for j in range(i + 1) if visible(i, j, m.get("mask"))]
        for hh in range(H):
            g = hh // (H // G)
            s = keys[js, g] @ q[t, hh] * m["scale"]
            out[t, hh] = sink_softmax(s, None if sink is None else float(sink[hh])) @ vals[js, g]
    out = out.reshape(T, H * dv) * sigmoid(h @ W[p + "g"].T)
    return out @ W[p + "o"].T


# ---- mixer M: state-space recurrence --------------------------------------------------------------------------------------------
def causal_conv(x, w, b, tail):
    """x [T, C], w [C, taps] (last column multiplies the current token), b [C], tail [taps-1, C] = the inputs before x.
    Returns (y [T, C], new tail)."""
    taps = w.shape[1]
    full = np.concatenate([tail, x], 0)
    y = np.zeros_like(x) + b[None, :]
    for j in range(taps):
        y += full[j:j + x.shape[0]] * w[:, j][None, :]
    return y, full[full.shape[0] - (taps - 1):].copy()


def ssm_scan(x, dt, a_log, B, C, D, S):
    """x [T, H, P]; dt [T, H]; a_log, D [H]; B, C [T, G, N]; S [H, N, P] is updated in place.  Returns y [T, H, P]."""
    T, H, P = x.shape
    G = B.shape[1]
    y = np.zeros((T, H, P))
    for t in range(T):
        for h in range(H):
            g = h // (H // G)
            S[h] = math.exp(-math.exp(a_log[h]) * dt[t, h]) * S[h] + dt[t, h] * np.outer(B[t, g], x[t, h])
            y[t, h] = S[h].T @ C[t, g] + D[h] * x[t, h]
    return y


def grouped_rms(y, parts, eps):
    T, n = y.shape
    return rms(y.reshape(T, parts, n // parts), eps).reshape(T, n)


def ssm_mixer(h, W, p, m, eps, state):
    """state: 'S' [heads, N, vdim] and 'tail' [taps-1, channels] (or empty at the start of a sequence)"""
    T = h.shape[0]
    H, P, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
    inner, gn = H * P, G * N
    proj = h @ W[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * gn], proj[:, 2 * inner + 2 * gn:]
    tail = state.get("tail", np.zeros((taps - 1, inner + 2 * gn)))
    xbc, state["tail"] = causal_conv(xbc, W[p + "conv"], W[p + "conv.b"], tail)
    xbc = silu(xbc)
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + gn].reshape(T, G, N)
    C = xbc[:, inner + gn:].reshape(T, G, N)
    dt = softplus(dt + W[p + "dt_bias"])
    if "S" not in state:
        state["S"] = np.zeros((H, N, P))
    y = ssm_scan(x, dt, W[p + "A_log"], B, C, W[p + "D"], state["S"]).reshape(T, inner)
    y = grouped_rms(y * silu(z), m.get("norm_groups", 1), eps) * W[p + "norm"]
    return y @ W[p + "o"].T


# ---- feed-forward ---------------------------------------------------------------------------------------------------------------
def dense_ff(h, W, p, f):
    lim = f.get("limit", math.inf)
    g = np.minimum(h @ W[p + "gate"].T, lim)
    u = np.clip(h @ W[p + "up"].T, -lim, lim)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


CHOICE_GAPS = []   # margin between the last chosen and the first rejected choice score of every routing decision made


def route(h, W, p, r):
    """-> (chosen [T, top] indices into experts + identity experts, weights [T, top])"""
    z = h @ W[p + "router"].T
    z = z - z.max(-1, keepdims=True)
    s = np.exp(z) / np.exp(z).sum(-1, keepdims=True)
    choice = s + (W[p + "correction"] if p + "correction" in W else 0.0)
    order = np.argsort(-choice, axis=-1, kind="stable")
    idx = order[:, :r["top"]]
    if choice.shape[1] > r["top"]:
        srt = np.take_along_axis(choice, order, -1)
        CHOICE_GAPS.extend((srt[:, r["top"] - 1] - srt[:, r["top"]]).tolist())
    sc = np.take_along_axis(s, idx, -1)
    return idx, sc / (sc.sum(-1, keepdims=True) + 1e-20)


def expert(h, W, p):
    return np.maximum(h @ W[p + "up"].T, 0.0) ** 2 @ W[p + "down"].T


def routed_ff(h, W, p, f):
    r = f["router"]
    E = r["experts"]
    idx, wts = route(h, W, p, r)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(idx[t], wts[t]):
            out[t] += w * (h[t] if e >= E else expert(h[t:t + 1], W, f"{p}e{e}.")[0])
    if f.get("shared"):
        out += expert(h, W, p + "shared.")
    return out


# ---- the model ----------------------------------------------------------------------------------------------------------------------------
class StepOracle:
    """Feeds tokens in portions; keeps every layer's state between calls."""

    def __init__(self, cfg, W):
        self.cfg, self.W = cfg, {k: np.asarray(v, np.float64) for k, v in W.items()}
        self.state = [dict() for _ in cfg["layers"]]
        self.pos = 0

    def step(self, tokens):
        """-> (logits [T, vocab], residual stream after every layer [layers, T, width])"""
        cfg, W, eps = self.cfg, self.W, self.cfg["norm"]["eps"]
        x = layer_norm(W["embed"][np.asarray(tokens, np.int64)], W["embed.norm"], eps)
        outs = []
        for i, L in enumerate(cfg["layers"]):
            p, m = f"l{i}.", L["mixer"]
            if L["type"] == "attention":
                y = attention_mixer(x, W, p + "mix.", m, eps, self.state[i], self.pos)
            elif L["type"] == "mamba2":
                y = ssm_mixer(x, W, p + "mix.", m, eps, self.state[i])
            else:
                raise ValueError(L["type"])
            x = x + W[p + "ls1"] * layer_norm(y, W[p + "norm1"], eps)
            f = L.get("mlp")
            if f:
                y = dense_ff(x, W, p + "mlp.", f) if f.get("kind", "dense") == "dense" else routed_ff(x, W, p + "mlp.", f)
                x = x + W[p + "ls2"] * layer_norm(y, W[p + "norm2"], eps)
            outs.append(x.copy())
        self.pos += len(tokens)
        logits = layer_norm(x, W["final.norm"], eps) @ W["head"].T * cfg.get("logit_scale", 1.0)
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
def dense(ff=56, limit=1.5):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts=5, identity=2, top=3, ff=24, shared=40):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


def attention_layer(heads=6, kv_heads=2, dim=12, vdim=20, size=9, keep_first=3, rot_dims=8, base=100.0, factor=2.0, scale=0.4, mlp="default"):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size:
        m["mask"] = {"size": size, "keep_first": keep_first}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
        if factor:
            m["rot"]["scaling"] = {"factor": factor}
    return {"type": "attention", "mixer": m, "mlp": moe() if mlp == "default" else mlp}


def ssm_layer(heads=4, vdim=10, state=12, groups=2, conv=4, norm_groups=2, mlp="default"):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups},
            "mlp": dense() if mlp == "default" else mlp}


def make_config(layers, width=40, vocab=70, eps=1e-5, logit_scale=0.5):
    return {"architecture": "Rupenex", "width": width, "vocab": vocab, "norm": {"eps": eps}, "logit_scale": logit_scale, "layers": layers}


def tensor_table(cfg):
    """[(name, shape, kind)]; kind: matrix | table | gain | scale | shift | conv | rate | zero"""
    w = cfg["width"]
    out = [("embed", (cfg["vocab"], w), "table"), ("embed.norm", (w,), "gain")]
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        q = p + "mix."
        out += [(p + "norm1", (w,), "gain"), (p + "ls1", (w,), "scale")]
        if L["type"] == "attention":
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out += [(q + "q", (H * dk, w), "matrix"), (q + "k", (G * dk, w), "matrix"), (q + "v", (G * dv, w), "matrix"),
                    (q + "q.norm", (dk,), "gain"), (q + "k.norm", (dk,), "gain"), (q + "sink", (H,), "shift"), (q + "g", (H * dv, w), "matrix"),
                    (q + "o", (w, H * dv), "matrix")]
        else:
            H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            inner, ch = H * P, H * P + 2 * G * N
            out += [(q + "in", (2 * inner + 2 * G * N + H, w), "matrix"), (q + "conv", (ch, m["conv"]), "conv"), (q + "conv.b", (ch,), "shift"),
                    (q + "dt_bias", (H,), "shift"), (q + "A_log", (H,), "rate"), (q + "D", (H,), "gain"), (q + "norm", (inner,), "gain"),
                    (q + "o", (w, inner), "matrix")]
        f = L.get("mlp")
        if f:
            out += [(p + "norm2", (w,), "gain"), (p + "ls2", (w,), "scale")]
            if f.get("kind", "dense") == "dense":
                out += [(p + "mlp.gate", (f["ff"], w), "matrix"), (p + "mlp.up", (f["ff"], w), "matrix"), (p + "mlp.down", (w, f["ff"]), "matrix")]
            else:
                r = f["router"]
                n = r["experts"] + r.get("identity", 0)
                out += [(p + "mlp.router", (n, w), "matrix"), (p + "mlp.correction", (n,), "zero")]
                for e in range(r["experts"]):
                    out += [(f"{p}mlp.e{e}.up", (f["expert"]["ff"], w), "matrix"), (f"{p}mlp.e{e}.down", (w, f["expert"]["ff"]), "matrix")]
                if f.get("shared"):
                    out += [(p + "mlp.shared.up", (f["shared"]["ff"], w), "matrix"), (p + "mlp.shared.down", (w, f["shared"]["ff"]), "matrix")]
    return out + [("final.norm", (w,), "gain"), ("head", (cfg["vocab"], w), "matrix")]


def random_weights(cfg, seed=0, gain=1.0):
    """bf16-representable float64 weights"""
    rng = np.random.default_rng(seed)
    W = {}
    for name, shape, kind in tensor_table(cfg):
        n = int(np.prod(shape)) if shape else 1
        if kind == "matrix":
            a = rng.standard_normal(n) * gain / math.sqrt(shape[-1])
            if name.endswith("router"):
                a *= 3.0
        elif kind == "table":
            a = rng.standard_normal(n)
        elif kind == "gain":
            a = 1.0 + 0.2 * rng.standard_normal(n)
        elif kind == "scale":
            a = 0.5 + 0.2 * rng.standard_normal(n)
        elif kind == "shift":
            a = 0.3 * rng.standard_normal(n)
        elif kind == "conv":
            a = rng.standard_normal(n) * 0.6
        elif kind == "rate":
            a = -1.0 + rng.standard_normal(n)
        else:
            a = 0.05 * rng.standard_normal(n)
        W[name] = bf16_round(a).reshape(shape)
    return W


def write_model(folder, cfg, W):
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
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
