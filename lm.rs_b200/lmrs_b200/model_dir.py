"""Model folders (config.json + model.safetensors) for the architectures the library opens by name: a writer, the
tensor tables of the Genetar, Tudatar, Rupenex and Badepel architectures, and random bf16 weights of a given shape for benchmarks and
smoke runs.

safetensors layout: 8-byte little-endian header length, that many bytes of JSON (name -> dtype, shape, data_offsets
relative to the end of the header), then the tensor data.
"""
import json
import math
import os
import struct

import numpy as np


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def genetar_config(width, ff, n_layers, heads, kv_heads, head_dim, vocab, *, buckets=4099, rot_dims=None, eps=1e-5,
                   softcap=50.0, logit_scale=1.0, pattern=("attention", "attention_2")):
    """layers alternate through `pattern`; every layer mixes values and has a dense SiLU-GLU feed-forward"""
    layers = []
    for i in range(n_layers):
        kind = pattern[i % len(pattern)]
        m = {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "scale": 1.0 / math.sqrt(head_dim),
             "softcap": softcap, "v_mix": True}
        if kind == "attention_2":
            m["rot"] = {"base": 500000.0, "dims": rot_dims or head_dim // 2,
                        "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}
        layers.append({"type": kind, "mixer": m, "mlp": {"kind": "dense", "ff": ff}})
    return {"architecture": "Genetar", "width": width, "vocab": vocab, "norm": {"eps": eps}, "logit_scale": logit_scale,
            "embedding": {"bigram": {"buckets": buckets, "mul_prev": 8191, "mul_cur": 127}}, "layers": layers}


def genetar_tensors(cfg):
    """[(name, shape, kind)]; kind: 'matrix' (fan-in scaled), 'table', 'ones', 'scalar'"""
    w, out = cfg["width"], [("embed", (cfg["vocab"], cfg["width"]), "table")]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        out.append(("bigram", (bg["buckets"] + 1, w), "table"))
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out += [(p + "norm1", (w,), "ones"), (p + "mix.q", (m["heads"] * m["dim"], w), "matrix"),
                (p + "mix.k", (m["kv_heads"] * m["dim"], w), "matrix"), (p + "mix.v", (m["kv_heads"] * m["vdim"], w), "matrix"),
                (p + "mix.vmix", (), "scalar")]
        if L["type"] == "attention_2":
            out.append((p + "mix.g", (m["heads"], w), "matrix"))
        out += [(p + "mix.o", (w, m["heads"] * m["vdim"]), "matrix"), (p + "ls1", (w,), "ones")]
        if L.get("mlp"):
            ff = L["mlp"]["ff"]
            out += [(p + "mlp.gate", (ff, w), "matrix"), (p + "mlp.up", (ff, w), "matrix"), (p + "mlp.down", (w, ff), "matrix"),
                    (p + "ls2", (w,), "ones")]
    out += [("final.norm", (w,), "ones"), ("head", (cfg["vocab"], w), "matrix")]
    return out


def genetar_param_bytes(cfg, bytes_per_weight=2):
    """bytes a decode step streams: every matrix once, one row of each table"""
    total = 0
    for name, shape, kind in genetar_tensors(cfg):
        n = int(np.prod(shape)) if shape else 1
        total += (shape[1] if kind == "table" else n) * bytes_per_weight
    return total


def genetar_matmul_flops_per_token(cfg):
    return sum(2 * int(np.prod(shape)) for name, shape, kind in genetar_tensors(cfg) if kind == "matrix")


def write_random(folder, cfg, table, seed=0):
    """random bf16 weights for a tensor table [(name, shape, kind)], streamed to disk tensor by tensor (a full-size model
    does not have to fit in host memory twice).  kind: matrix (fan-in scaled) | table | ones | scalar | shift | conv | rate |
    small | zero | decay | read | write | mixing"""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, off = {}, 0
    for name, shape, _ in table:
        n = (int(np.prod(shape)) if shape else 1) * 2
        header[name] = {"dtype": "BF16", "shape": list(shape), "data_offsets": [off, off + n]}
        off += n
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    rng = np.random.default_rng(seed)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj)
        for name, shape, kind in table:
            n = int(np.prod(shape)) if shape else 1
            if kind == "ones":
                a = 1.0 + 0.1 * rng.standard_normal(n, dtype=np.float32)
            elif kind == "scalar":
                a = np.array([0.25], np.float32)
            elif kind == "alpha":
                a = np.array([0.5], np.float32)
            elif kind == "shift":
                a = 0.1 * rng.standard_normal(n, dtype=np.float32)
            elif kind == "conv":
                a = 0.5 * rng.standard_normal(n, dtype=np.float32)
            elif kind == "rate":
                a = -1.0 + 0.5 * rng.standard_normal(n, dtype=np.float32)
            elif kind == "small":
                a = (0.05 + 0.2 * rng.random(n)).astype(np.float32)
            elif kind == "zero":
                a = 0.05 * rng.standard_normal(n, dtype=np.float32)
            elif kind == "decay":   # logits of decays close to one
                a = 3.0 + rng.standard_normal(n, dtype=np.float32)
            elif kind == "read":    # stream weights: a sublayer reads about the mean of the streams, ...
                a = (1.0 / shape[0] + 0.1 * rng.standard_normal(n)).astype(np.float32)
            elif kind == "write":   # ... writes to all of them, ...
                a = 1.0 + 0.2 * rng.standard_normal(n, dtype=np.float32)
            elif kind == "mixing":  # ... and the streams mix a little among themselves
                a = (np.eye(shape[0]) + 0.05 * rng.standard_normal(shape)).astype(np.float32).reshape(-1)
            else:
                a = rng.standard_normal(n, dtype=np.float32)
                if kind == "matrix":
                    a *= np.float32(1.0 / math.sqrt(shape[-1]))
            f.write(f32_to_bf16_bits(a).tobytes())
    return folder


def write_random_genetar(folder, cfg, seed=0):
    return write_random(folder, cfg, genetar_tensors(cfg), seed)


# ---- Tudatar ---------------------------------------------------------------------------------------------------------------
def tudatar_config(width, n_layers, vocab, *, heads=16, kv_heads=4, head_dim=64, window=1024, delta_heads=None, delta_dim=None,
                   conv=4, kv_rank=256, q_rank=768, rot_dim=64, experts=16, top=4, expert_ff=2048, eps=1e-5, logit_scale=1.0,
                   pattern=("channel_delta", "attention", "channel_delta", "latent_attention"), low_rank=64):
    """layers cycle through `pattern`; every layer has a routed-expert feed-forward (experts == 0: none)"""
    layers = []
    mlp = {"kind": "moe", "expert": {"ff": expert_ff}, "router": {"experts": experts, "top": top, "scale": 1.0}} if experts else None
    for i in range(n_layers):
        kind = pattern[i % len(pattern)]
        if kind == "channel_delta":
            h = delta_heads or heads
            d = delta_dim or head_dim
            m = {"heads": h, "kv_heads": h, "dim": d, "vdim": d, "conv": conv, "a_rank": low_rank, "g_rank": low_rank}
        elif kind == "latent_attention":
            m = {"heads": heads, "dim": head_dim, "rot_dim": rot_dim, "vdim": head_dim, "kv_rank": kv_rank, "q_rank": q_rank,
                 "scale": 1.0 / math.sqrt(head_dim + rot_dim),
                 "rot": {"base": 10000.0, "dims": rot_dim, "scaling": {"factor": 8.0, "fast": 32.0, "slow": 1.0, "original": 4096}}}
        else:
            m = {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "scale": 1.0 / math.sqrt(head_dim),
                 "mask": {"size": window}}
        layers.append({"type": kind, "mixer": m, "mlp": mlp})
    return {"architecture": "Tudatar", "width": width, "vocab": vocab, "norm": {"eps": eps}, "logit_scale": logit_scale, "layers": layers}


def tudatar_tensors(cfg):
    """[(name, shape, kind)] -- the ranks of the delta rule's two low-rank projections are tensor shapes, not configuration:
    the writer takes them from the hints a_rank / g_rank that tudatar_config leaves in the mixer entry"""
    w = cfg["width"]

    def norm(n):
        return [(n, (w,), "ones"), (n + ".b", (w,), "shift"), (n + ".alpha", (), "alpha")]
    out = [("embed", (cfg["vocab"], w), "table")]
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out += norm(p + "norm1") + norm(p + "norm1b")
        q = p + "mix."
        if L["type"] == "channel_delta":
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            ra, rg = m.get("a_rank", 64), m.get("g_rank", 64)
            out += [(q + "q", (G * dk, w), "matrix"), (q + "q.conv", (G * dk, m["conv"]), "conv"), (q + "k", (G * dk, w), "matrix"),
                    (q + "k.conv", (G * dk, m["conv"]), "conv"), (q + "v", (H * dv, w), "matrix"), (q + "v.conv", (H * dv, m["conv"]), "conv"),
                    (q + "b", (H, w), "matrix"), (q + "A_log", (H,), "rate"), (q + "norm", (dv,), "ones"), (q + "a1", (ra, w), "matrix"),
                    (q + "a2", (H * dk, ra), "matrix"), (q + "dt_bias", (H * dk,), "shift"), (q + "g1", (rg, w), "matrix"),
                    (q + "g2", (H * dv, rg), "matrix"), (q + "o", (w, H * dv), "matrix")]
        elif L["type"] == "latent_attention":
            H, dn, dr, dv, rk, rq = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            out += [(q + "dq", (rq, w), "matrix"), (q + "dq.norm", (rq,), "ones"), (q + "uq", (H * (dn + dr), rq), "matrix"),
                    (q + "dkv", (rk + dr, w), "matrix"), (q + "dkv.norm", (rk,), "ones"), (q + "uk", (H * dn, rk), "matrix"),
                    (q + "uv", (H * dv, rk), "matrix"), (q + "o", (w, H * dv), "matrix")]
        else:
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out += [(q + "q", (H * dk, w), "matrix"), (q + "q.b", (H * dk,), "shift"), (q + "k", (G * dk, w), "matrix"),
                    (q + "k.b", (G * dk,), "shift"), (q + "v", (G * dv, w), "matrix"), (q + "v.b", (G * dv,), "shift"),
                    (q + "q.norm", (H * dk,), "ones"), (q + "k.norm", (G * dk,), "ones"), (q + "r1", (H,), "small"), (q + "r2", (H,), "small"),
                    (q + "o", (w, H * dv), "matrix")]
        if L.get("mlp"):
            f = L["mlp"]
            out += norm(p + "norm2") + norm(p + "norm2b")
            out += [(p + "mlp.router", (f["router"]["experts"], w), "matrix"), (p + "mlp.correction", (f["router"]["experts"],), "zero")]
            for e in range(f["router"]["experts"]):
                out += [(f"{p}mlp.e{e}.gate", (f["expert"]["ff"], w), "matrix"), (f"{p}mlp.e{e}.up", (f["expert"]["ff"], w), "matrix"),
                        (f"{p}mlp.e{e}.down", (w, f["expert"]["ff"]), "matrix")]
    return out + norm("final.norm") + [("head", (cfg["vocab"], w), "matrix")]


def _tudatar_active(cfg, name):
    """share of a tensor that one token touches: an expert matrix counts top / experts"""
    if ".mlp.e" in name:
        f = cfg["layers"][int(name[1:name.index(".")])]["mlp"]["router"]
        return f["top"] / f["experts"]
    return 1.0


def tudatar_param_bytes(cfg, bytes_per_weight=2):
    """bytes a decode step streams: every matrix of the mixers once, the chosen experts, one row of the embedding table"""
    total = 0.0
    for name, shape, kind in tudatar_tensors(cfg):
        n = int(np.prod(shape)) if shape else 1
        total += (shape[1] if kind == "table" else n) * bytes_per_weight * _tudatar_active(cfg, name)
    return int(total)


def tudatar_matmul_flops_per_token(cfg):
    return int(sum(2 * int(np.prod(shape)) * _tudatar_active(cfg, name) for name, shape, kind in tudatar_tensors(cfg) if kind == "matrix"))


def tudatar_mixer_flops(cfg, T):
    """FLOPs of the sequence mixers' cores over a prompt of T tokens: attention (in the latent space for latent layers, inside the
    window for windowed ones) and the delta-rule scan (two passes over the state per token)"""
    total = 0
    for L in cfg["layers"]:
        m = L["mixer"]
        if L["type"] == "channel_delta":
            total += 6 * m["heads"] * m["dim"] * m["vdim"] * T
        elif L["type"] == "latent_attention":
            total += 2 * m["heads"] * (2 * m["kv_rank"] + m["rot_dim"]) * T * (T + 1) // 2
        else:
            w = m.get("mask", {}).get("size", 0) or T
            pairs = T * (T + 1) // 2 if T <= w else w * (w + 1) // 2 + (T - w) * w
            total += 2 * m["heads"] * (m["dim"] + m["vdim"]) * pairs
    return total


def write_random_tudatar(folder, cfg, seed=0):
    return write_random(folder, cfg, tudatar_tensors(cfg), seed)


# ---- Rupenex ---------------------------------------------------------------------------------------------------------------
def rupenex_config(width, n_layers, vocab, *, heads=16, kv_heads=4, head_dim=64, window=1024, keep_first=4, rot_dims=None, ssm_heads=None,
                   ssm_vdim=64, state=128, groups=8, conv=4, norm_groups=8, ff=8192, experts=16, identity=2, top=4, expert_ff=2048,
                   shared_ff=2048, limit=7.0, eps=1e-5, logit_scale=1.0, pattern=("mamba2", "attention"), mlps=("dense", "moe")):
    """layers cycle through `pattern`, their feed-forwards through `mlps` (dense | moe | None); a state-space layer's inner size
    is 2 * width unless ssm_heads says otherwise"""
    layers = []
    for i in range(n_layers):
        kind, fk = pattern[i % len(pattern)], mlps[i % len(mlps)]
        if kind == "mamba2":
            m = {"heads": ssm_heads or 2 * width // ssm_vdim, "vdim": ssm_vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}
        else:
            m = {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "scale": 1.0 / math.sqrt(head_dim),
                 "mask": {"size": window, "keep_first": keep_first},
                 "rot": {"base": 500000.0, "dims": rot_dims or head_dim, "scaling": {"factor": 8.0}}}
        if fk == "dense":
            f = {"kind": "dense", "ff": ff, "limit": limit}
        elif fk == "moe":
            f = {"kind": "moe", "expert": {"ff": expert_ff}, "router": {"experts": experts, "identity": identity, "top": top}}
            if shared_ff:
                f["shared"] = {"ff": shared_ff}
        else:
            f = None
        layers.append({"type": kind, "mixer": m, "mlp": f})
    return {"architecture": "Rupenex", "width": width, "vocab": vocab, "norm": {"eps": eps}, "logit_scale": logit_scale, "layers": layers}


def rupenex_tensors(cfg):
    w = cfg["width"]
    out = [("embed", (cfg["vocab"], w), "table"), ("embed.norm", (w,), "ones")]
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        q = p + "mix."
        out += [(p + "norm1", (w,), "ones"), (p + "ls1", (w,), "small")]
        if L["type"] == "attention":
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out += [(q + "q", (H * dk, w), "matrix"), (q + "k", (G * dk, w), "matrix"), (q + "v", (G * dv, w), "matrix"), (q + "q.norm", (dk,), "ones"),
                    (q + "k.norm", (dk,), "ones"), (q + "sink", (H,), "shift"), (q + "g", (H * dv, w), "matrix"), (q + "o", (w, H * dv), "matrix")]
        else:
            H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            inner, ch = H * P, H * P + 2 * G * N
            out += [(q + "in", (2 * inner + 2 * G * N + H, w), "matrix"), (q + "conv", (ch, m["conv"]), "conv"), (q + "conv.b", (ch,), "shift"),
                    (q + "dt_bias", (H,), "shift"), (q + "A_log", (H,), "rate"), (q + "D", (H,), "ones"), (q + "norm", (inner,), "ones"),
                    (q + "o", (w, inner), "matrix")]
        f = L.get("mlp")
        if f:
            out += [(p + "norm2", (w,), "ones"), (p + "ls2", (w,), "small")]
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
    return out + [("final.norm", (w,), "ones"), ("head", (cfg["vocab"], w), "matrix")]


def _rupenex_active(cfg, name):
    """share of a tensor that one token touches: a routed expert's matrix counts top / (experts + identity experts), which is what a
    uniform router sends its way"""
    if ".mlp.e" in name:
        r = cfg["layers"][int(name[1:name.index(".")])]["mlp"]["router"]
        return r["top"] / (r["experts"] + r.get("identity", 0))
    return 1.0


def rupenex_param_bytes(cfg, bytes_per_weight=2):
    """bytes a decode step streams: every matrix of the mixers and dense layers once, the chosen experts, one embedding row"""
    total = 0.0
    for name, shape, kind in rupenex_tensors(cfg):
        n = int(np.prod(shape)) if shape else 1
        total += (shape[1] if kind == "table" else n) * bytes_per_weight * _rupenex_active(cfg, name)
    return int(total)


def rupenex_matmul_flops_per_token(cfg):
    return int(sum(2 * int(np.prod(shape)) * _rupenex_active(cfg, name) for name, shape, kind in rupenex_tensors(cfg) if kind == "matrix"))


def rupenex_mixer_flops(cfg, T):
    """FLOPs of the sequence mixers' cores over a prompt of T tokens: attention inside the window (plus the kept first keys) and
    the state-space scan (update and read-out of the state per token)"""
    total = 0
    for L in cfg["layers"]:
        m = L["mixer"]
        if L["type"] == "mamba2":
            total += 6 * m["heads"] * m["state"] * m["vdim"] * T
        else:
            w = (m.get("mask") or {}).get("size", 0) or T
            pairs = T * (T + 1) // 2 if T <= w else w * (w + 1) // 2 + (T - w) * (w + (m.get("mask") or {}).get("keep_first", 0))
            total += 2 * m["heads"] * (m["dim"] + m["vdim"]) * pairs
    return total


def write_random_rupenex(folder, cfg, seed=0):
    return write_random(folder, cfg, rupenex_tensors(cfg), seed)


# ---- Badepel ---------------------------------------------------------------------------------------------------------------
def badepel_config(width, n_layers, vocab, *, streams=4, residual_mult=0.5, heads=16, kv_heads=4, head_dim=64, window=1024, rot_dims=None,
                   conv=4, softcap=30.0, gla_heads=None, gla_dim=64, gla_vdim=64, gla_rank=64, tau=8.0, delta_heads=None, delta_kv_heads=None,
                   delta_dim=64, delta_vdim=64, ff=8192, experts=16, top=4, expert_ff=2048, shared_ff=2048, limit=7.0, eps=1e-5,
                   pattern=("delta", "parallel"), mlps=("dense", "moe")):
    """layers cycle through `pattern`, their feed-forwards through `mlps` (dense | moe | None); the inner size of the
    recurrent mixers is the model width unless their head counts say otherwise"""
    layers = []
    for i in range(n_layers):
        kind, fk = pattern[i % len(pattern)], mlps[i % len(mlps)]
        if kind == "delta":
            h = delta_heads or width // delta_vdim
            m = {"heads": h, "kv_heads": delta_kv_heads or h, "dim": delta_dim, "vdim": delta_vdim, "conv": conv}
        else:
            left = {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "conv": conv, "scale": 1.0 / math.sqrt(head_dim),
                    "softcap": softcap, "mask": {"size": window}, "rot": {"base": 500000.0, "dims": rot_dims or head_dim}}
            right = {"heads": gla_heads or width // gla_vdim, "dim": gla_dim, "vdim": gla_vdim, "tau": tau, "rank": gla_rank}
            m = {"left": left, "right": right, "left_scale": 1.0, "right_scale": 1.0}
        if fk == "dense":
            f = {"kind": "dense", "ff": ff}
        elif fk == "moe":
            f = {"kind": "moe", "expert": {"ff": expert_ff, "limit": limit}, "router": {"experts": experts, "top": top}}
            if shared_ff:
                f["shared"] = {"ff": shared_ff, "limit": limit}
        else:
            f = None
        layers.append({"type": kind, "mixer": m, "mlp": f})
    return {"architecture": "Badepel", "width": width, "vocab": vocab, "norm": {"eps": eps}, "streams": streams, "residual_mult": residual_mult,
            "layers": layers}


def badepel_tensors(cfg):
    """[(name, shape, kind)] -- the rank of the right mixer's decay projection is a tensor shape, not configuration: the writer
    takes it from the hint `rank` that badepel_config leaves in the mixer entry"""
    w, S = cfg["width"], cfg.get("streams", 1)
    out = [("embed", (cfg["vocab"], w), "table")]
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        q = p + "mix."
        out += [(p + "norm1", (w,), "ones")]
        if L["type"] == "parallel":
            l, r = m["left"], m["right"]
            H, G, dk, dv = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
            for n, rows in (("q", H * dk), ("k", G * dk), ("v", G * dv)):
                out += [(f"{q}left.{n}", (rows, w), "matrix"), (f"{q}left.{n}.b", (rows,), "shift")]
                if l.get("conv"):
                    out.append((f"{q}left.{n}.conv", (rows, l["conv"]), "conv"))
            out += [(q + "left.q.norm", (H * dk,), "ones"), (q + "left.k.norm", (G * dk,), "ones"), (q + "left.o", (w, H * dv), "matrix")]
            Hr, dkr, dvr, ra = r["heads"], r["dim"], r["vdim"], r.get("rank", 16)
            out += [(q + "right.q", (Hr * dkr, w), "matrix"), (q + "right.k", (Hr * dkr, w), "matrix"), (q + "right.v", (Hr * dvr, w), "matrix"),
                    (q + "right.g", (Hr * dvr, w), "matrix"), (q + "right.o", (w, Hr * dvr), "matrix"), (q + "right.norm", (dvr,), "ones"),
                    (q + "right.a1", (ra, w), "matrix"), (q + "right.a2", (Hr * dkr, ra), "matrix"), (q + "right.a2.b", (Hr * dkr,), "decay")]
        else:
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for n, rows in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                out += [(q + n, (rows, w), "matrix"), (q + n + ".conv", (rows, m["conv"]), "conv")]
            out += [(q + "b", (H, w), "matrix"), (q + "A_log", (H,), "rate"), (q + "norm", (dv,), "ones"), (q + "a", (H, w), "matrix"),
                    (q + "dt_bias", (H,), "shift"), (q + "g", (H * dv, w), "matrix"), (q + "o", (w, H * dv), "matrix")]
        f = L.get("mlp")
        if f:
            out += [(p + "norm2", (w,), "ones")]
            if f.get("kind", "dense") == "dense":
                out += [(p + "mlp.gate", (f["ff"], w), "matrix"), (p + "mlp.up", (f["ff"], w), "matrix"), (p + "mlp.down", (w, f["ff"]), "matrix")]
            else:
                r, ff = f["router"], f["expert"]["ff"]
                for e in range(r["experts"]):
                    out += [(f"{p}mlp.e{e}.gate", (ff, w), "matrix"), (f"{p}mlp.e{e}.up", (ff, w), "matrix"), (f"{p}mlp.e{e}.down", (w, ff), "matrix")]
                out += [(p + "mlp.router", (r["experts"], w), "matrix"), (p + "mlp.router.b", (r["experts"],), "shift")]
                if f.get("shared"):
                    sf = f["shared"]["ff"]
                    out += [(p + "mlp.shared.gate", (sf, w), "matrix"), (p + "mlp.shared.up", (sf, w), "matrix"), (p + "mlp.shared.down", (w, sf), "matrix")]
        for s in ("hc1", "hc2") if f else ("hc1",):
            out += [(f"{p}{s}.in", (S,), "read"), (f"{p}{s}.out", (S,), "write"), (f"{p}{s}.mix", (S, S), "mixing")]
    return out + [("final.norm", (w,), "ones"), ("head", (cfg["vocab"], w), "matrix")]


def _badepel_active(cfg, name):
    """share of a tensor that one token touches: a routed expert's matrix counts top / experts"""
    if ".mlp.e" in name:
        r = cfg["layers"][int(name[1:name.index(".")])]["mlp"]["router"]
        return r["top"] / r["experts"]
    return 1.0


def badepel_param_bytes(cfg, bytes_per_weight=2):
    """bytes a decode step streams: every matrix of the mixers and dense layers once, the chosen experts, one embedding row"""
    total = 0.0
    for name, shape, kind in badepel_tensors(cfg):
        n = int(np.prod(shape)) if shape else 1
        total += (shape[1] if kind == "table" else n) * bytes_per_weight * _badepel_active(cfg, name)
    return int(total)


def badepel_matmul_flops_per_token(cfg):
    return int(sum(2 * int(np.prod(shape)) * _badepel_active(cfg, name) for name, shape, kind in badepel_tensors(cfg) if kind == "matrix"))


def badepel_mixer_flops(cfg, T):
    """FLOPs of the sequence mixers' cores over a prompt of T tokens: attention inside the window, the gated-linear-attention
    scan (update and read-out of the state per token) and the delta-rule scan (two passes over the state per token)"""
    total = 0
    for L in cfg["layers"]:
        m = L["mixer"]
        if L["type"] == "delta":
            total += 6 * m["heads"] * m["dim"] * m["vdim"] * T
        else:
            l, r = m["left"], m["right"]
            w = (l.get("mask") or {}).get("size", 0) or T
            pairs = T * (T + 1) // 2 if T <= w else w * (w + 1) // 2 + (T - w) * w
            total += 2 * l["heads"] * (l["dim"] + l["vdim"]) * pairs + 5 * r["heads"] * r["dim"] * r["vdim"] * T
    return total


def written_badepel_config(cfg):
    """config.json without the writer's hints"""
    c = json.loads(json.dumps(cfg))
    for L in c["layers"]:
        if L["type"] == "parallel":
            L["mixer"]["right"].pop("rank", None)
    return c


def write_random_badepel(folder, cfg, seed=0):
    write_random(folder, cfg, badepel_tensors(cfg), seed)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(written_badepel_config(cfg), f)
    return folder
