// mixer_ops.cuh -- what happens between a sequence mixer's input projection and its core, for the mixers that are not plain
// multi-head attention, and the one core that is not attention (dense_ops.cuh has the attention kernel):
//   latent_kv_post_kernel     attention through a shared latent: RMS norm of the query latent and of the key/value latent,
//                             pairwise rotation of the shared rotated key part, latent + rotated part written to the cache
//   latent_q_post_kernel      per query head: unrotated part to the operand type (it is multiplied into the latent space
//                             next), rotated part rotated and placed behind the latent-space part of the query; or, for the
//                             per-head form, the whole head [unrotated | rotated] in f32
//   latent_expand_kernel      per-head keys [up-projected latent | shared rotated part] assembled for all cached positions
//   qkv_jointnorm_post_kernel q and k RMS-normalised over the WHOLE projection (all heads at once) with a weight, v divided
//                             by its root mean square per head (or kept); optionally a short causal convolution in front
//                             and a pairwise rotation behind; k and v written to the cache
//   delta_pre_kernel          gated delta rule: short causal convolution + SiLU on q, k, v channels (continued from a tail of
//                             earlier inputs), unit-length q and k per head, write strength sigmoid
//   conv_tail_update_kernel   the last taps-1 inputs of every channel become the tail for the next step
//   delta_scan_kernel         S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q, token after token, the
//                             state matrix of a head spread over the registers of the threads that own its columns; with one
//                             decay per head instead of per key channel; or without the correction (gated linear attention:
//                             S <- diag(g) S + k v^T)
//   gated_headnorm_kernel     o / rms(o) * w * sigmoid(gate) per head, in the operand type
//   ssm_pre_kernel            state-space recurrence with one decay per head: short causal convolution + bias + SiLU over the
//                             (x, B, C) channels, step sizes dt = softplus(raw + bias) and decays exp(-exp(A_log) dt)
//   ssm_scan_kernel           S <- decay S + dt B x^T;  y = S^T C + D x, token after token, same thread layout as the
//                             delta-rule scan
//   gated_groupnorm_kernel    (y * silu(z)) / rms over each of `groups` equal parts of the row, * w, in the operand type
// Everything here is f32 (positions, angles, norms, decays, the recurrent state); only rows that feed the next matrix
// product are written in the operand type.
#pragma once
#include "dense_ops.cuh"

namespace lmrs {
namespace dense {

// first rot_dims entries of an n-vector rotated pairwise -- (2i, 2i+1) by the angle of cos[i], sin[i] -- the rest copied; one warp
DN_DEVINL void rotate_pairs_warp(const float* src, float* dst, int n, int rot_dims, const float* c, const float* s, int lane) {
    for (int i = lane; i < rot_dims / 2; i += 32) {
        const float u = src[2 * i], v = src[2 * i + 1];
        dst[2 * i] = u * c[i] - v * s[i];
        dst[2 * i + 1] = v * c[i] + u * s[i];
    }
    for (int d = rot_dims + lane; d < n; d += 32) dst[d] = src[d];
}

// ---- attention through a latent: the projected row [query latent (rq) | key/value latent (rk) | rotated key part (dr)] ----
template <typename AT> struct LatentKvPostParams {
    const float* in; int ld;
    int rq, rk, dr;
    const float* wq; const float* wkv; float eps;                 // norm weights of the two latents
    int rot_dims; const float* rot_cos; const float* rot_sin;      // [max_tokens][rot_dims/2], multiplier folded in
    AT* cq_out;                                                   // [T][rq]
    float* cache;                                                 // [max_tokens][rk + dr]
    AT* cache_op;                                                 // [max_tokens][rk]: the latent again, in the operand type
    PosSrc ps;
};
template <typename AT> __global__ void __launch_bounds__(256) latent_kv_post_kernel(const LatentKvPostParams<AT> p) {
    __shared__ float red[33];
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    const uint32_t pos = pos_of(p.ps) + (uint32_t)t;
    const float* row = p.in + (size_t)t * p.ld;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < p.rq; c += blockDim.x) ss += row[c] * row[c];
    ss = block_sum(ss, red);
    float inv = 1.0f / sqrtf(ss / (float)p.rq + p.eps);
    for (int c = threadIdx.x; c < p.rq; c += blockDim.x) from_f(p.cq_out[(size_t)t * p.rq + c], row[c] * inv * p.wq[c]);
    const float* kv = row + p.rq;
    ss = 0.0f;
    for (int c = threadIdx.x; c < p.rk; c += blockDim.x) ss += kv[c] * kv[c];
    ss = block_sum(ss, red);
    inv = 1.0f / sqrtf(ss / (float)p.rk + p.eps);
    float* dst = p.cache + (size_t)pos * (p.rk + p.dr);
    for (int c = threadIdx.x; c < p.rk; c += blockDim.x) {
        const float v = kv[c] * inv * p.wkv[c];
        dst[c] = v;
        from_f(p.cache_op[(size_t)pos * p.rk + c], v);
    }
    if (threadIdx.x < 32) {
        const int half = p.rot_dims / 2;
        rotate_pairs_warp(kv + p.rk, dst + p.rk, p.dr, p.rot_dims, p.rot_cos + (size_t)pos * half, p.rot_sin + (size_t)pos * half, threadIdx.x);
    }
}

template <typename AT> struct LatentQPostParams {
    const float* q;           // [T][H * (dn + dr)], head by head [unrotated | rotated]
    int H, dn, dr, rk;
    int rot_dims; const float* rot_cos; const float* rot_sin;
    AT* qn_out;               // [T][H * dn]
    float* qabs;              // [T][H * (rk + dr)]: the rotated part goes to columns rk .. rk+dr of each head
    float* qfull;             // when set instead: [T][H * (dn + dr)], the unrotated part copied, the rotated part rotated
    PosSrc ps;
};
template <typename AT> __global__ void __launch_bounds__(128) latent_q_post_kernel(const LatentQPostParams<AT> p) {
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x, lane = threadIdx.x & 31;
    const int h = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (h >= p.H) return;
    const uint32_t pos = pos_of(p.ps) + (uint32_t)t;
    const float* src = p.q + ((size_t)t * p.H + h) * (p.dn + p.dr);
    const int half = p.rot_dims / 2;
    if (p.qfull) {
        float* dst = p.qfull + ((size_t)t * p.H + h) * (p.dn + p.dr);
        for (int d = lane; d < p.dn; d += 32) dst[d] = src[d];
        rotate_pairs_warp(src + p.dn, dst + p.dn, p.dr, p.rot_dims, p.rot_cos + (size_t)pos * half, p.rot_sin + (size_t)pos * half, lane);
        return;
    }
    AT* qn = p.qn_out + ((size_t)t * p.H + h) * p.dn;
    for (int d = lane; d < p.dn; d += 32) from_f(qn[d], src[d]);
    rotate_pairs_warp(src + p.dn, p.qabs + ((size_t)t * p.H + h) * (p.rk + p.dr) + p.rk, p.dr, p.rot_dims,
                      p.rot_cos + (size_t)pos * half, p.rot_sin + (size_t)pos * half, lane);
}

// keys per head for positions 0 .. n: kfull[j][h] = [knope[j][h] (dn) | cached rotated part of position j (dr)]
struct LatentExpandParams {
    const float* knope;       // [n][H * dn] up-projected latents
    const float* cache;       // [max_tokens][rk + dr]
    float* kfull;             // [n][H * (dn + dr)]
    int H, dn, dr, rk;
};
static __global__ void __launch_bounds__(256) latent_expand_kernel(const LatentExpandParams p) {
    pdl_launch();
    pdl_wait();
    const int j = blockIdx.x, dq = p.dn + p.dr;
    const float* kr = p.cache + (size_t)j * (p.rk + p.dr) + p.rk;
    for (int e = threadIdx.x; e < p.H * dq; e += blockDim.x) {
        const int h = e / dq, d = e - h * dq;
        p.kfull[(size_t)j * p.H * dq + e] = d < p.dn ? p.knope[((size_t)j * p.H + h) * p.dn + d] : kr[d - p.dn];
    }
}

// ---- q and k normalised over the whole projection, v per head --------------------------------------------------------------
// Optional steps, each off when its parameter is zero / null:
//   taps > 0     a short causal convolution over time on every channel of [q | k | v] right after the projection (taps [C][taps],
//                last tap on the current token, no activation), continued from a tail [taps-1][C] of earlier inputs as in
//                conv_input below; the convolved row of q or k is staged in dynamic shared memory (max(H, G) * dk floats)
//   rot_dims > 0 after the norm, the first rot_dims dimensions of every q and k head are rotated in neighbouring pairs
//                (2i, 2i+1) by the angle of cos/sin[position][i]
//   v_plain      the values are cached as they are instead of being divided by their root mean square per head
constexpr int CONV_MAX_TAPS = 16;
DN_DEVINL float conv_input(const float* in, int ld, const float* tail, int C, int taps, int tq, int c, uint32_t pos0) {
    if (tq >= 0) return in[(size_t)tq * ld + c];
    if ((long long)pos0 + tq < 0) return 0.0f;
    return tail[(size_t)(taps - 1 + tq) * C + c];
}
struct QkvJointNormParams {
    const float* qkv; int ld;   // [q (H*dk) | k (G*dk) | v (G*dv)], biases already added
    int H, G, dk, dv;
    const float* wq; const float* wk; float eps;
    float* q_out;               // [T][H*dk]
    float* kcache; float* vcache;
    PosSrc ps;
    int taps; const float* wconv; const float* tail;             // convolution over the C = (H+G)*dk + G*dv channels
    int rot_dims; const float* rot_cos; const float* rot_sin;    // [max_tokens][rot_dims/2]
    int v_plain;
    float* tail_out;            // set (to the tail) for a step of one token (THREADS > 256): the thread that convolves a channel also moves its tail on
};
// grid (T, 3): q, k and v of a token; block size up to THREADS (a one-token step takes 1024: its rows are all the work there is)
template <int THREADS> __global__ void __launch_bounds__(THREADS) qkv_jointnorm_post_kernel(const QkvJointNormParams p) {
    extern __shared__ __align__(16) float jn_row[];
    __shared__ float red[33];
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    const uint32_t pos0 = pos_of(p.ps), pos = pos0 + (uint32_t)t;
    const float* row = p.qkv + (size_t)t * p.ld;
    const int nq = p.H * p.dk, nk = p.G * p.dk, C = nq + nk + p.G * p.dv;
    auto conv = [&](int c) {   // channel c of this token after the convolution
        float a = 0.0f;
#pragma unroll 4
        for (int j = 0; j < p.taps; j++) a = fmaf(p.wconv[(size_t)c * p.taps + j], conv_input(p.qkv, p.ld, p.tail, C, p.taps, t - (p.taps - 1 - j), c, pos0), a);
        return a;
    };
    auto move_tail = [&](int c) {   // the last taps-1 inputs of channel c become its tail (this thread alone touches the channel)
        float nv[CONV_MAX_TAPS];
#pragma unroll
        for (int r = 0; r < CONV_MAX_TAPS; r++)
            if (r < p.taps - 1) nv[r] = conv_input(p.qkv, p.ld, p.tail, C, p.taps, (int)gridDim.x - (p.taps - 1) + r, c, pos0);
#pragma unroll
        for (int r = 0; r < CONV_MAX_TAPS; r++)
            if (r < p.taps - 1) p.tail_out[(size_t)r * C + c] = nv[r];
    };
    if (blockIdx.y < 2) {
        const bool is_q = blockIdx.y == 0;
        const int c0 = is_q ? 0 : nq;
        const float* src = row + c0;
        const int n = is_q ? nq : nk;
        const float* w = is_q ? p.wq : p.wk;
        float* dst = is_q ? p.q_out + (size_t)t * nq : p.kcache + (size_t)pos * nk;
        float ss = 0.0f;
        if (p.taps > 0) {
            for (int c = threadIdx.x; c < n; c += blockDim.x) { const float v = conv(c0 + c); jn_row[c] = v; ss += v * v; }
            if (THREADS > 256 && p.tail_out)   // (the one-token form only: the small-block form stays lean)
                for (int c = threadIdx.x; c < n; c += blockDim.x) move_tail(c0 + c);
            src = jn_row;
        } else {
            for (int c = threadIdx.x; c < n; c += blockDim.x) ss += src[c] * src[c];
        }
        ss = block_sum(ss, red);   // (its barriers also order the staged row before the reads below)
        const float inv = 1.0f / sqrtf(ss / (float)n + p.eps);
        if (p.rot_dims > 0) {
            const int half = p.rot_dims / 2;
            const float* cs = p.rot_cos + (size_t)pos * half;
            const float* sn = p.rot_sin + (size_t)pos * half;
            for (int c = threadIdx.x; c < n; c += blockDim.x) {
                const int d = c % p.dk;
                const float v = src[c] * inv * w[c];
                if (d >= p.rot_dims) { dst[c] = v; continue; }
                const int cp = c - d + (d ^ 1);                // rot_dims is even: the partner is in the same head
                const float o = src[cp] * inv * w[cp];
                dst[c] = (d & 1) ? v * cs[d >> 1] + o * sn[d >> 1] : v * cs[d >> 1] - o * sn[d >> 1];
            }
        } else {
            for (int c = threadIdx.x; c < n; c += blockDim.x) dst[c] = src[c] * inv * w[c];
        }
        return;
    }
    const int lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int g = threadIdx.x >> 5; g < p.G; g += nw) {
        const int c0 = nq + nk + g * p.dv;
        const float* src = row + c0;
        float* dst = p.vcache + ((size_t)pos * p.G + g) * p.dv;
        if (p.v_plain) {
            for (int d = lane; d < p.dv; d += 32) dst[d] = p.taps > 0 ? conv(c0 + d) : src[d];
            if (THREADS > 256 && p.tail_out)
                for (int d = lane; d < p.dv; d += 32) move_tail(c0 + d);
            continue;
        }
        float ss = 0.0f;
        for (int d = lane; d < p.dv; d += 32) { const float v = p.taps > 0 ? conv(c0 + d) : src[d]; ss += v * v; }
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)p.dv + p.eps);
        for (int d = lane; d < p.dv; d += 32) dst[d] = (p.taps > 0 ? conv(c0 + d) : src[d]) * inv;
        if (THREADS > 256 && p.tail_out)
            for (int d = lane; d < p.dv; d += 32) move_tail(c0 + d);
    }
}

// ---- gated delta rule -------------------------------------------------------------------------------------------------------------
// The projected row is [q (G*dk) | k (G*dk) | v (H*dv) | write-strength logits (H) | decay latent (ra) | gate latent (rg)].
// Its first C = 2*G*dk + H*dv entries are the convolution's channels, in the order of the tail [taps-1][C] and of the taps
// [C][taps] (last tap = current token).  An input before the sequence's start is zero; one before this step's first row
// comes from the tail.
template <typename AT> struct DeltaPreParams {
    const float* in; int ld;
    int H, G, dk, dv, taps, ra, rg;
    const float* wconv;       // [C][taps]
    const float* tail;        // [taps-1][C]
    float* qkv_out;           // [T][C]: q (unit length / sqrt(dk)), k (unit length), v
    float* beta;              // [T][H]
    AT* a_lat; AT* g_lat;     // [T][ra], [T][rg]: operands of the second halves of the two low-rank projections
    PosSrc ps;
    // one decay per head instead of the low-rank projection (ra = 0): the H columns behind the write-strength logits are decay
    // logits, head_decay[t][h] = exp(-exp(a_log[h]) * softplus(logit + dt_bias[h]))
    float* head_decay; const float* a_log; const float* dt_bias;
};
template <typename AT> __global__ void __launch_bounds__(128) delta_pre_kernel(const DeltaPreParams<AT> p) {
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    const uint32_t pos0 = pos_of(p.ps);
    const int lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int wid = blockIdx.y * nw + (threadIdx.x >> 5), wtotal = gridDim.y * nw;
    const int nqk = 2 * p.G, nv = p.H * p.dv, C = nqk * p.dk + nv, v_tasks = (nv + 127) / 128;
    const float* row = p.in + (size_t)t * p.ld;
    float* out = p.qkv_out + (size_t)t * C;
    auto conv_silu = [&](int c) {
        float a = 0.0f;
        for (int j = 0; j < p.taps; j++) a = fmaf(p.wconv[(size_t)c * p.taps + j], conv_input(p.in, p.ld, p.tail, C, p.taps, t - (p.taps - 1 - j), c, pos0), a);
        return silu(a);
    };
    for (int task = wid; task < nqk + v_tasks + 1; task += wtotal) {
        if (task < nqk) {   // one q or k head: convolution, SiLU, unit length (q also / sqrt(dk))
            const int c0 = task * p.dk;
            float ss = 0.0f;
            for (int d = lane; d < p.dk; d += 32) { const float v = conv_silu(c0 + d); out[c0 + d] = v; ss += v * v; }
            ss = warp_sum(ss);
            const float inv = (task < p.G ? 1.0f / sqrtf((float)p.dk) : 1.0f) / sqrtf(ss + 1e-6f);
            for (int d = lane; d < p.dk; d += 32) out[c0 + d] *= inv;   // a lane rescales what it wrote itself
        } else if (task < nqk + v_tasks) {
            const int c0 = nqk * p.dk, i0 = (task - nqk) * 128, i1 = min(nv, i0 + 128);
            for (int i = i0 + lane; i < i1; i += 32) out[c0 + i] = conv_silu(c0 + i);
        } else {
            for (int h = lane; h < p.H; h += 32) p.beta[(size_t)t * p.H + h] = 1.0f / (1.0f + expf(-row[C + h]));
            if (p.head_decay)
                for (int h = lane; h < p.H; h += 32) {
                    const float a = row[C + p.H + h] + p.dt_bias[h];
                    p.head_decay[(size_t)t * p.H + h] = expf(-expf(p.a_log[h]) * (a > 20.0f ? a : log1pf(expf(a))));
                }
            for (int i = lane; i < p.ra; i += 32) from_f(p.a_lat[(size_t)t * p.ra + i], row[C + p.H + i]);
            for (int i = lane; i < p.rg; i += 32) from_f(p.g_lat[(size_t)t * p.rg + i], row[C + p.H + p.ra + i]);
        }
    }
}
struct ConvTailParams {
    const float* in; int ld;
    float* tail; int C, taps, T;
    PosSrc ps;
};
static __global__ void __launch_bounds__(256) conv_tail_update_kernel(const ConvTailParams p) {
    pdl_launch();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= p.C) return;
    const uint32_t pos0 = pos_of(p.ps);
    float nv[CONV_MAX_TAPS];
#pragma unroll
    for (int r = 0; r < CONV_MAX_TAPS; r++)
        if (r < p.taps - 1) nv[r] = conv_input(p.in, p.ld, p.tail, p.C, p.taps, p.T - (p.taps - 1) + r, c, pos0);
#pragma unroll
    for (int r = 0; r < CONV_MAX_TAPS; r++)
        if (r < p.taps - 1) p.tail[(size_t)r * p.C + c] = nv[r];
}

// decay per (token, head, key channel) from the projected logits, in place: g = exp(-exp(a_log[head]) * softplus(logit)), or,
// without a_log, g = sigmoid(logit)^(1/tau) = exp(-softplus(-logit) / tau)
struct DeltaDecayParams {
    float* a;              // [T][H*dk] logits in, decays out
    const float* a_log;    // [H] or null
    int n, H, dk;          // n = T * H * dk
    float inv_tau;
};
static __global__ void __launch_bounds__(256) delta_decay_kernel(const DeltaDecayParams p) {
    pdl_launch();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.n) return;
    const float a = p.a_log ? p.a[i] : -p.a[i];
    const float sp = a > 20.0f ? a : log1pf(expf(a));
    p.a[i] = p.a_log ? expf(-expf(p.a_log[(i / p.dk) % p.H]) * sp) : expf(-sp * p.inv_tau);
}

// The scan.  CTA = (block of state columns, head); a column j of the head's state S [dk][dv] belongs to `lpc` adjacent lanes,
// lane s of them holding NR rows in registers: groups of four consecutive rows, group r4 at rows (r4*lpc + s)*4 .., so a
// lane reads its q, k and decay entries of a token with 16-byte shared-memory loads that do not collide with its neighbours'.
// Columns never interact: S^T k and S^T q are sums down a column, the rank-one update adds k_i u_j.  Tokens are staged
// DELTA_TB at a time in shared memory by cp.async (q, k, decays, v, beta), the next block in flight while this one is used;
// rows beyond dk are zero-filled, so the arithmetic needs no bounds.  Every token costs two passes over the registers and two
// reductions across the lpc lanes.  The order of every sum is fixed, so a token's result does not depend on the portion it
// arrives in.  The state is read at the start (zeros when the step starts at position 0) and written back at the end.
constexpr int DELTA_TB = 8, DELTA_THREADS = 128, DELTA_MAX_DK = 512;
struct DeltaScanParams {
    const float* qkv; int ld;   // [T][C]: q at 0, k at G*dk, v at 2*G*dk
    const float* decay;         // [T][H*dk]
    const float* beta;          // [T][H]
    float* state;               // [H][dk][dv]
    float* out;                 // [T][H*dv]
    int T, H, G, dk, dv;
    PosSrc ps;
    float q_scale;              // the read-out times this constant (0: none)
};
// what the scan computes per token.  SCAN_DELTA: the rule above with a decay per key channel.  SCAN_DELTA_HEAD: the same with
// one decay per head (decay is [T][H]).  SCAN_PLAIN: no correction and no write strength, S <- diag(g) S + k v^T, o = S^T q
// (gated linear attention): one pass over the registers and one lane reduction per token.
enum { SCAN_DELTA = 0, SCAN_DELTA_HEAD = 1, SCAN_PLAIN = 2 };
// (rows per lane NR, lanes per column LPC) for a key size: NR * LPC >= dk.  A warp issues dependent instructions only every few
// cycles, so the split favours many lanes per column (more warps per scheduler, shorter chains) over few
inline void delta_scan_shape(int dk, int* nr, int* lpc) {
    if (dk <= 16) { *nr = 16; *lpc = 1; }
    else if (dk <= 32) { *nr = 16; *lpc = 2; }
    else if (dk <= 64) { *nr = 8; *lpc = 8; }
    else if (dk <= 128) { *nr = 8; *lpc = 16; }
    else if (dk <= 256) { *nr = 8; *lpc = 32; }
    else { *nr = 16; *lpc = 32; }
}
inline size_t delta_scan_smem(int nr, int lpc) { return (size_t)2 * DELTA_TB * (3 * nr * lpc + DELTA_THREADS / lpc + 4) * 4; }
DN_DEVINL void cp_async4_zfill(void* smem_dst, const void* gsrc, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const int n = valid ? 4 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(gsrc), "r"(n) : "memory");
}
template <int NR, int LPC, int MODE = SCAN_DELTA> __global__ void __launch_bounds__(DELTA_THREADS) delta_scan_kernel(const DeltaScanParams p) {
    extern __shared__ __align__(16) float ds_sm[];
    pdl_launch();
    pdl_wait();
    constexpr int cols = DELTA_THREADS / LPC, dkp = NR * LPC;   // dkp: rows the lanes cover (>= dk, a multiple of 4)
    constexpr int blk = DELTA_TB * (3 * dkp + cols + 4);                   // floats per staging buffer
    const int h = blockIdx.y, g = h / (p.H / p.G);
    const int s = threadIdx.x % LPC, jl = threadIdx.x / LPC, j = blockIdx.x * cols + jl;
    const bool col_ok = j < p.dv;
    const uint32_t pos0 = pos_of(p.ps);
    const int vq = 2 * p.G * p.dk;
    // 16-byte copies when every row piece starts on a 16-byte boundary
    const bool vec = (p.dk & 3) == 0 && (p.ld & 3) == 0 && ((p.H * p.dk) & 3) == 0 && (reinterpret_cast<uintptr_t>(p.qkv) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(p.decay) & 15) == 0;
    auto stage = [&](int t0, int buf) {
        float* qs = ds_sm + (size_t)buf * blk;     // [TB][dkp]
        float* ks = qs + DELTA_TB * dkp;
        float* gs = ks + DELTA_TB * dkp;
        float* vs = gs + DELTA_TB * dkp;           // [TB][cols]
        float* bs = vs + DELTA_TB * cols;          // [TB]
        const int nt = min(DELTA_TB, p.T - t0);
        if (vec) {
            const int q4 = dkp >> 2;
            for (int e = threadIdx.x; e < nt * q4; e += blockDim.x) {
                const int tt = e / q4, i = (e - tt * q4) << 2;
                const bool ok = i < p.dk;
                const float* row = p.qkv + (size_t)(t0 + tt) * p.ld;
                cp_async16_zfill(qs + tt * dkp + i, ok ? row + g * p.dk + i : p.qkv, ok);
                cp_async16_zfill(ks + tt * dkp + i, ok ? row + (p.G + g) * p.dk + i : p.qkv, ok);
                if (MODE != SCAN_DELTA_HEAD) cp_async16_zfill(gs + tt * dkp + i, ok ? p.decay + ((size_t)(t0 + tt) * p.H + h) * p.dk + i : p.qkv, ok);
            }
        } else {
            for (int e = threadIdx.x; e < nt * dkp; e += blockDim.x) {
                const int tt = e / dkp, i = e - tt * dkp;
                const bool ok = i < p.dk;
                const float* row = p.qkv + (size_t)(t0 + tt) * p.ld;
                cp_async4_zfill(qs + tt * dkp + i, ok ? row + g * p.dk + i : p.qkv, ok);
                cp_async4_zfill(ks + tt * dkp + i, ok ? row + (p.G + g) * p.dk + i : p.qkv, ok);
                if (MODE != SCAN_DELTA_HEAD) cp_async4_zfill(gs + tt * dkp + i, ok ? p.decay + ((size_t)(t0 + tt) * p.H + h) * p.dk + i : p.qkv, ok);
            }
        }
        for (int e = threadIdx.x; e < nt * cols; e += blockDim.x) {
            const int tt = e / cols, c = e - tt * cols, jj = blockIdx.x * cols + c;
            cp_async4_zfill(vs + e, jj < p.dv ? p.qkv + (size_t)(t0 + tt) * p.ld + vq + h * p.dv + jj : p.qkv, jj < p.dv);
        }
        if (MODE != SCAN_PLAIN && threadIdx.x < nt) cp_async4_zfill(bs + threadIdx.x, p.beta + (size_t)(t0 + threadIdx.x) * p.H + h, true);
        if (MODE == SCAN_DELTA_HEAD && threadIdx.x < nt) cp_async4_zfill(gs + threadIdx.x, p.decay + (size_t)(t0 + threadIdx.x) * p.H + h, true);   // gs[tt]: the head's decay
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    stage(0, 0);
    float S[NR];
    float* sp = p.state + ((size_t)h * p.dk) * p.dv + j;
#pragma unroll
    for (int r = 0; r < NR; r++) {
        const int i = ((r >> 2) * LPC + s) * 4 + (r & 3);
        S[r] = (pos0 > 0 && col_ok && i < p.dk) ? sp[(size_t)i * p.dv] : 0.0f;
    }
    int buf = 0;
    for (int t0 = 0; t0 < p.T; t0 += DELTA_TB, buf ^= 1) {
        const int nt = min(DELTA_TB, p.T - t0);
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();   // this block has landed for everyone, and everyone is done with the other buffer
        if (t0 + DELTA_TB < p.T) stage(t0 + DELTA_TB, buf ^ 1);
        const float* qs = ds_sm + (size_t)buf * blk;
        const float* ks = qs + DELTA_TB * dkp;
        const float* gs = ks + DELTA_TB * dkp;
        const float* vs = gs + DELTA_TB * dkp;
        const float* bs = vs + DELTA_TB * cols;
        for (int tt = 0; tt < nt; tt++) {
            float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
            if (MODE == SCAN_PLAIN) {
                const float u = vs[tt * cols + jl];
#pragma unroll
                for (int r4 = 0; r4 < NR / 4; r4++) {
                    const int i = (r4 * LPC + s) * 4;
                    const float4 g4 = *reinterpret_cast<const float4*>(gs + tt * dkp + i);
                    const float4 k4 = *reinterpret_cast<const float4*>(ks + tt * dkp + i);
                    const float4 q4 = *reinterpret_cast<const float4*>(qs + tt * dkp + i);
                    S[4 * r4] = fmaf(S[4 * r4], g4.x, k4.x * u); S[4 * r4 + 1] = fmaf(S[4 * r4 + 1], g4.y, k4.y * u);
                    S[4 * r4 + 2] = fmaf(S[4 * r4 + 2], g4.z, k4.z * u); S[4 * r4 + 3] = fmaf(S[4 * r4 + 3], g4.w, k4.w * u);
                    o0 = fmaf(S[4 * r4], q4.x, o0); o1 = fmaf(S[4 * r4 + 1], q4.y, o1);
                    o2 = fmaf(S[4 * r4 + 2], q4.z, o2); o3 = fmaf(S[4 * r4 + 3], q4.w, o3);
                }
            } else {
            float kk[NR];
            float r0 = 0.0f, r1 = 0.0f, r2 = 0.0f, r3 = 0.0f;
            const float gh = MODE == SCAN_DELTA_HEAD ? gs[tt] : 1.0f;
#pragma unroll
            for (int r4 = 0; r4 < NR / 4; r4++) {
                const int i = (r4 * LPC + s) * 4;
                const float4 g4 = MODE == SCAN_DELTA_HEAD ? make_float4(gh, gh, gh, gh) : *reinterpret_cast<const float4*>(gs + tt * dkp + i);
                const float4 k4 = *reinterpret_cast<const float4*>(ks + tt * dkp + i);
                kk[4 * r4] = k4.x; kk[4 * r4 + 1] = k4.y; kk[4 * r4 + 2] = k4.z; kk[4 * r4 + 3] = k4.w;
                S[4 * r4] *= g4.x; S[4 * r4 + 1] *= g4.y; S[4 * r4 + 2] *= g4.z; S[4 * r4 + 3] *= g4.w;
                r0 = fmaf(S[4 * r4], k4.x, r0); r1 = fmaf(S[4 * r4 + 1], k4.y, r1);
                r2 = fmaf(S[4 * r4 + 2], k4.z, r2); r3 = fmaf(S[4 * r4 + 3], k4.w, r3);
            }
            float rsum = (r0 + r1) + (r2 + r3);
            for (int o = LPC >> 1; o > 0; o >>= 1) rsum += __shfl_xor_sync(0xffffffffu, rsum, o);
            const float u = bs[tt] * (vs[tt * cols + jl] - rsum);
#pragma unroll
            for (int r4 = 0; r4 < NR / 4; r4++) {
                const int i = (r4 * LPC + s) * 4;
                const float4 q4 = *reinterpret_cast<const float4*>(qs + tt * dkp + i);
                S[4 * r4] = fmaf(kk[4 * r4], u, S[4 * r4]); S[4 * r4 + 1] = fmaf(kk[4 * r4 + 1], u, S[4 * r4 + 1]);
                S[4 * r4 + 2] = fmaf(kk[4 * r4 + 2], u, S[4 * r4 + 2]); S[4 * r4 + 3] = fmaf(kk[4 * r4 + 3], u, S[4 * r4 + 3]);
                o0 = fmaf(S[4 * r4], q4.x, o0); o1 = fmaf(S[4 * r4 + 1], q4.y, o1);
                o2 = fmaf(S[4 * r4 + 2], q4.z, o2); o3 = fmaf(S[4 * r4 + 3], q4.w, o3);
            }
            }
            float osum = (o0 + o1) + (o2 + o3);
            for (int o = LPC >> 1; o > 0; o >>= 1) osum += __shfl_xor_sync(0xffffffffu, osum, o);
            if (p.q_scale != 0.0f) osum *= p.q_scale;
            if (s == 0 && col_ok) p.out[(size_t)(t0 + tt) * p.H * p.dv + (size_t)h * p.dv + j] = osum;
        }
    }
    if (col_ok) {
#pragma unroll
        for (int r = 0; r < NR; r++) {
            const int i = ((r >> 2) * LPC + s) * 4 + (r & 3);
            if (i < p.dk) sp[(size_t)i * p.dv] = S[r];
        }
    }
}

// o / sqrt(mean(o^2) + eps) * w[c] * sigmoid(gate logit) per (token, head): one warp each
// gate_silu: the gate is silu(logit) instead.  g_ld / out_ld (with H): the gate logits / the output of a token are H * dv
// columns of a wider row with this pitch; has_out_scale: the output times out_scale
template <typename AT> struct GatedHeadNormParams {
    const float* o; const float* graw;   // [rows][dv] each, rows = T * H
    const float* w; float eps;
    AT* out;
    int rows, dv;
    int gate_silu, H, g_ld, out_ld, has_out_scale;
    float out_scale;
};
template <typename AT> __global__ void __launch_bounds__(128) gated_headnorm_kernel(const GatedHeadNormParams<AT> p) {
    pdl_launch();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= p.rows) return;
    const float* o = p.o + (size_t)r * p.dv;
    const int t = p.H > 0 ? r / p.H : 0, hh = p.H > 0 ? r % p.H : 0;
    const float* gr = p.g_ld > 0 ? p.graw + (size_t)t * p.g_ld + (size_t)hh * p.dv : p.graw + (size_t)r * p.dv;
    AT* dst = p.out_ld > 0 ? p.out + (size_t)t * p.out_ld + (size_t)hh * p.dv : p.out + (size_t)r * p.dv;
    float ss = 0.0f;
    for (int c = lane; c < p.dv; c += 32) ss += o[c] * o[c];
    ss = warp_sum(ss);
    const float inv = (p.has_out_scale ? p.out_scale : 1.0f) / sqrtf(ss / (float)p.dv + p.eps);
    for (int c = lane; c < p.dv; c += 32) {
        const float sg = 1.0f / (1.0f + expf(-gr[c]));
        from_f(dst[c], o[c] * inv * p.w[c] * (p.gate_silu ? gr[c] * sg : sg));
    }
}

// ---- state-space recurrence with a scalar decay per head --------------------------------------------------------------------
// The projected row holds, among others, the convolution's C channels (from column c_off: x [H*P] | B [G*N] | C [G*N]) and
// the raw step sizes (H columns from dt_off).  Convolution as above: taps [C][taps] with the last tap on the current token,
// a tail [taps-1][C] of earlier inputs, zeros before the sequence's start; then + bias and SiLU.  A thread owns one channel
// for a run of SSM_PRE_TT tokens, so its taps stay in registers and a warp's loads are contiguous; a step of at most
// SSM_PRE_TT tokens also moves the tail on here (longer steps leave that to conv_tail_update_kernel, which runs after every
// block has read the old tail).  The last block column computes dt = softplus(raw + dt_bias[h]) and decay = exp(-exp(a_log[h]) * dt) for its tokens, all in f32.
constexpr int SSM_PRE_TT = 16;
struct SsmPreParams {
    const float* in; int ld;
    int c_off, C, taps;
    const float* wconv; const float* bconv; const float* tail;
    float* out;               // [T][C]
    int dt_off, H;
    const float* dt_bias; const float* a_log;
    float* dt; float* decay;  // [T][H]
    int T;
    float* tail_out;          // set (to the tail) when the grid has one block of tokens: the kernel then also moves the tail on
    PosSrc ps;
};
static __global__ void __launch_bounds__(128) ssm_pre_kernel(const SsmPreParams p) {
    pdl_launch();
    pdl_wait();
    const uint32_t pos0 = pos_of(p.ps);
    const int t0 = blockIdx.y * SSM_PRE_TT, t1 = min(p.T, t0 + SSM_PRE_TT);
    if (blockIdx.x == gridDim.x - 1) {
        for (int e = threadIdx.x; e < (t1 - t0) * p.H; e += blockDim.x) {
            const int t = t0 + e / p.H, h = e % p.H;
            const float a = p.in[(size_t)t * p.ld + p.dt_off + h] + p.dt_bias[h];
            const float dt = a > 20.0f ? a : log1pf(expf(a));
            p.dt[(size_t)t * p.H + h] = dt;
            p.decay[(size_t)t * p.H + h] = expf(-expf(p.a_log[h]) * dt);
        }
        return;
    }
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= p.C) return;
    float w[CONV_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; j++) w[j] = j < p.taps ? p.wconv[(size_t)c * p.taps + j] : 0.0f;
    const float b = p.bconv ? p.bconv[c] : 0.0f;
    const float* in = p.in + p.c_off;
    for (int t = t0; t < t1; t++) {
        float a = b;
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; j++)
            if (j < p.taps) a = fmaf(w[j], conv_input(in, p.ld, p.tail, p.C, p.taps, t - (p.taps - 1 - j), c, pos0), a);
        p.out[(size_t)t * p.C + c] = silu(a);
    }
    if (p.tail_out) {   // this thread is the only one that touches channel c: the new tail is the last taps-1 inputs
        float nv[CONV_MAX_TAPS];
#pragma unroll
        for (int r = 0; r < CONV_MAX_TAPS; r++)
            if (r < p.taps - 1) nv[r] = conv_input(in, p.ld, p.tail, p.C, p.taps, p.T - (p.taps - 1) + r, c, pos0);
#pragma unroll
        for (int r = 0; r < CONV_MAX_TAPS; r++)
            if (r < p.taps - 1) p.tail_out[(size_t)r * p.C + c] = nv[r];
    }
}

// The scan.  CTA = (block of state columns, head); a column j (one of the head's P value channels) of the state S [N][P]
// belongs to `lpc` adjacent lanes, lane s of them holding NR rows in registers, in the row order of delta_scan_kernel so
// that B and C entries are read with 16-byte shared-memory loads; a thread may own CPT adjacent columns, which share those reads.  Per token and row: S <- decay * S + (dt x_j) B_i, and
// y_j += S C_i; one reduction across the lpc lanes, then + D x_j.  Tokens are staged DELTA_TB at a time by cp.async, the
// next block in flight while this one is used.  The order of every sum is fixed, so a token's result does not depend on the
// portion it arrives in.  The state is read at the start (zeros when the step starts at position 0) and written back at
// the end.
struct SsmScanParams {
    const float* xbc; int ld;   // [T][C]: x of head h at h*P, B of group g at b_off + g*N, C at c_off + g*N
    int b_off, c_off;
    const float* dt; const float* decay;   // [T][H]
    const float* D;                        // [H]
    float* state;                          // [H][N][P]
    float* out;                            // [T][H*P]
    int T, H, G, N, P;
    PosSrc ps;
};
inline size_t ssm_scan_smem(int nr, int lpc, int cpt) { return (size_t)2 * DELTA_TB * (2 * nr * lpc + cpt * DELTA_THREADS / lpc + 2) * 4; }
template <int NR, int LPC, int CPT> __global__ void __launch_bounds__(DELTA_THREADS) ssm_scan_kernel(const SsmScanParams p) {
    extern __shared__ __align__(16) float ss_sm[];
    pdl_launch();
    pdl_wait();
    // a thread owns CPT adjacent columns: one read of a token's B and C entries then serves CPT columns
    constexpr int cols = DELTA_THREADS / LPC * CPT, dkp = NR * LPC;
    constexpr int blk = DELTA_TB * (2 * dkp + cols + 2);
    const int h = blockIdx.y, g = h / (p.H / p.G);
    const int s = threadIdx.x % LPC, jl = threadIdx.x / LPC * CPT, j = blockIdx.x * cols + jl;
    const uint32_t pos0 = pos_of(p.ps);
    const bool vec = (p.N & 3) == 0 && (p.ld & 3) == 0 && (p.b_off & 3) == 0 && (p.c_off & 3) == 0;
    auto stage = [&](int t0, int buf) {
        float* bs = ss_sm + (size_t)buf * blk;     // [TB][dkp]
        float* cs = bs + DELTA_TB * dkp;
        float* xs = cs + DELTA_TB * dkp;           // [TB][cols]
        float* dts = xs + DELTA_TB * cols;         // [TB]
        float* des = dts + DELTA_TB;               // [TB]
        const int nt = min(DELTA_TB, p.T - t0);
        if (vec) {
            const int q4 = dkp >> 2;
            for (int e = threadIdx.x; e < nt * q4; e += blockDim.x) {
                const int tt = e / q4, i = (e - tt * q4) << 2;
                const bool ok = i < p.N;
                const float* row = p.xbc + (size_t)(t0 + tt) * p.ld;
                cp_async16_zfill(bs + tt * dkp + i, ok ? row + p.b_off + g * p.N + i : p.xbc, ok);
                cp_async16_zfill(cs + tt * dkp + i, ok ? row + p.c_off + g * p.N + i : p.xbc, ok);
            }
        } else {
            for (int e = threadIdx.x; e < nt * dkp; e += blockDim.x) {
                const int tt = e / dkp, i = e - tt * dkp;
                const bool ok = i < p.N;
                const float* row = p.xbc + (size_t)(t0 + tt) * p.ld;
                cp_async4_zfill(bs + tt * dkp + i, ok ? row + p.b_off + g * p.N + i : p.xbc, ok);
                cp_async4_zfill(cs + tt * dkp + i, ok ? row + p.c_off + g * p.N + i : p.xbc, ok);
            }
        }
        for (int e = threadIdx.x; e < nt * cols; e += blockDim.x) {
            const int tt = e / cols, c = e - tt * cols, jj = blockIdx.x * cols + c;
            cp_async4_zfill(xs + e, jj < p.P ? p.xbc + (size_t)(t0 + tt) * p.ld + h * p.P + jj : p.xbc, jj < p.P);
        }
        if (threadIdx.x < nt) {
            cp_async4_zfill(dts + threadIdx.x, p.dt + (size_t)(t0 + threadIdx.x) * p.H + h, true);
            cp_async4_zfill(des + threadIdx.x, p.decay + (size_t)(t0 + threadIdx.x) * p.H + h, true);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    stage(0, 0);
    float S[CPT][NR];
    float* sp = p.state + ((size_t)h * p.N) * p.P + j;
#pragma unroll
    for (int cc = 0; cc < CPT; cc++)
#pragma unroll
        for (int r = 0; r < NR; r++) {
            const int i = ((r >> 2) * LPC + s) * 4 + (r & 3);
            S[cc][r] = (pos0 > 0 && j + cc < p.P && i < p.N) ? sp[(size_t)i * p.P + cc] : 0.0f;
        }
    const float dskip = p.D ? p.D[h] : 0.0f;
    int buf = 0;
    for (int t0 = 0; t0 < p.T; t0 += DELTA_TB, buf ^= 1) {
        const int nt = min(DELTA_TB, p.T - t0);
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();   // this block has landed for everyone, and everyone is done with the other buffer
        if (t0 + DELTA_TB < p.T) stage(t0 + DELTA_TB, buf ^ 1);
        const float* bs = ss_sm + (size_t)buf * blk;
        const float* cs = bs + DELTA_TB * dkp;
        const float* xs = cs + DELTA_TB * dkp;
        const float* dts = xs + DELTA_TB * cols;
        const float* des = dts + DELTA_TB;
        for (int tt = 0; tt < nt; tt++) {
            const float a = des[tt], dtv = dts[tt];
            float xv[CPT], dtx[CPT], y[CPT][4];
#pragma unroll
            for (int cc = 0; cc < CPT; cc++) {
                xv[cc] = xs[tt * cols + jl + cc];
                dtx[cc] = dtv * xv[cc];
                y[cc][0] = y[cc][1] = y[cc][2] = y[cc][3] = 0.0f;
            }
#pragma unroll
            for (int r4 = 0; r4 < NR / 4; r4++) {
                const int i = (r4 * LPC + s) * 4;
                const float4 b4 = *reinterpret_cast<const float4*>(bs + tt * dkp + i);
                const float4 c4 = *reinterpret_cast<const float4*>(cs + tt * dkp + i);
                const float bv[4] = {b4.x, b4.y, b4.z, b4.w}, cv[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
                for (int cc = 0; cc < CPT; cc++)
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        S[cc][4 * r4 + k] = fmaf(a, S[cc][4 * r4 + k], dtx[cc] * bv[k]);
                        y[cc][k] = fmaf(S[cc][4 * r4 + k], cv[k], y[cc][k]);
                    }
            }
#pragma unroll
            for (int cc = 0; cc < CPT; cc++) {
                float ysum = (y[cc][0] + y[cc][1]) + (y[cc][2] + y[cc][3]);
                for (int o = LPC >> 1; o > 0; o >>= 1) ysum += __shfl_xor_sync(0xffffffffu, ysum, o);
                if (s == 0 && j + cc < p.P) p.out[(size_t)(t0 + tt) * p.H * p.P + (size_t)h * p.P + j + cc] = fmaf(dskip, xv[cc], ysum);
            }
        }
    }
#pragma unroll
    for (int cc = 0; cc < CPT; cc++)
#pragma unroll
        for (int r = 0; r < NR; r++) {
            const int i = ((r >> 2) * LPC + s) * 4 + (r & 3);
            if (j + cc < p.P && i < p.N) sp[(size_t)i * p.P + cc] = S[cc][r];
        }
}

// v = y * silu(z); the row is cut into `groups` equal parts, each divided by its own root mean square (eps inside the root),
// then * w[column]: one CTA per (token, part)
template <typename AT> struct GatedGroupNormParams {
    const float* y; int ldy;
    const float* z; int ldz;
    const float* w; float eps;
    AT* out; int ldo;
    int n, groups;
};
template <typename AT> __global__ void __launch_bounds__(256) gated_groupnorm_kernel(const GatedGroupNormParams<AT> p) {
    __shared__ float red[33];
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x, gs = p.n / p.groups, c0 = blockIdx.y * gs;
    const float* y = p.y + (size_t)t * p.ldy + c0;
    const float* z = p.z + (size_t)t * p.ldz + c0;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < gs; c += blockDim.x) { const float v = y[c] * silu(z[c]); ss += v * v; }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)gs + p.eps);
    for (int c = threadIdx.x; c < gs; c += blockDim.x) from_f(p.out[(size_t)t * p.ldo + c0 + c], y[c] * silu(z[c]) * inv * p.w[c0 + c]);
}

}  // namespace dense
}  // namespace lmrs
