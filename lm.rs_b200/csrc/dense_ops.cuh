// dense_ops.cuh -- kernels for models with unquantized weights (bf16 or f32 operands, f32 accumulation): the building
// blocks a folder-based architecture (arch.h) composes.  Every constant of a mechanism is a parameter, so that another
// architecture can use the same kernel:
//   embed_rows_kernel        token embedding + optional hashed bigram embedding of (previous token, token)
//   rmsnorm_rows_kernel      x / sqrt(mean(x^2) + eps) * w per row, optional row gather, output in the operand type
//   tanhnorm_rows_kernel     tanh(alpha * x) * w + b per element (a norm without statistics), same gather and output
//   layernorm_rows_kernel    (x - mean) / sqrt(var + eps) * w per row; the result is stored, or scaled per column and added
//                            to the residual stream, and the row that comes out is also written in the operand type
//   gemv_rows_kernel         one token row:  weights streamed once (HBM-bound), optional fused RMS-norm prologue,
//                            epilogues: store*scale+bias | x += ls * f(acc) + lb | act(gate) * up | store in the operand
//                            type; a batch dimension (per-head matrices, or experts picked by a device-side index list)
//   gemm_tiled_kernel        many rows, any shape, CUDA cores (the f32 path and ragged shapes); same epilogues; batched
//                            over column blocks (one matrix per head) or grouped over row ranges (one matrix per expert)
//   qkv_post_kernel          per head: unit RMS norm of q/k or partial rotary, value mixing with an earlier layer's
//                            values, sigmoid head gate, K/V rows written to the cache
//   attn_rows_kernel         causal softmax attention with score scale and tanh soft-cap, optional sliding window (with
//                            first positions that stay visible), logarithmic distance penalty, a learned per-head sink
//                            in the softmax denominator, per-head or per-element sigmoid output gates, grouped query
//                            heads, query tile x KV head per CTA, K and V rows
//                            with their own pitch (V may be a prefix of the K row: attention over a shared latent),
//                            optional split over the keys (decode) + attn_combine_kernel
// What the design wants in 32-bit (norms, scores, softmax, residual, angles) is 32-bit here in both operand types.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "step_params.h"

namespace lmrs {
namespace dense {

#define DN_DEVINL __device__ __forceinline__

DN_DEVINL float to_f(float v) { return v; }
DN_DEVINL float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
DN_DEVINL void from_f(float& d, float v) { d = v; }
DN_DEVINL void from_f(__nv_bfloat16& d, float v) { d = __float2bfloat16_rn(v); }

DN_DEVINL float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
DN_DEVINL float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// sum over the block (blockDim.x a multiple of 32, <= 1024); every thread gets the result; `red` = 33 floats of smem
DN_DEVINL float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? red[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    const float r = red[32];
    __syncthreads();
    return r;
}

// Programmatic dependent launch: a kernel launched with the attribute may start while its predecessor in the stream is
// still running; pdl_wait() blocks until the predecessor has completed and its writes are visible (a no-op without the
// attribute), pdl_launch() lets the successor start its own pre-wait part now.  Every kernel here waits before it touches
// anything but weights, so a chain of them stays ordered.
DN_DEVINL void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
DN_DEVINL void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// position of row 0 of a step: a host constant, or read from the device-resident step parameters (decode graphs)
struct PosSrc {
    const StepParams* sp;
    uint32_t pos;
};
DN_DEVINL uint32_t pos_of(const PosSrc& s) { return s.sp ? s.sp->pos : s.pos; }

// ---- embedding -----------------------------------------------------------------------------------------------------
// x[t] = embed[token] + bigram[(prev * mul_prev + token * mul_cur) mod buckets]; the first token of a sequence takes the
// extra row `buckets`.  The token history lives on the device (tokens[position]): the previous token of a portion's
// first row is whatever the previous step left there.
template <typename WT> struct EmbedRowsParams {
    const WT* embed; const WT* bigram;   // bigram may be null
    uint32_t* tokens;                    // [max_tokens] history, rows pos .. pos+T-1 already filled for sp == null
    float* x; int width;
    PosSrc ps;
    uint32_t buckets, mul_prev, mul_cur;
};
template <typename WT> __global__ void __launch_bounds__(128) embed_rows_kernel(const EmbedRowsParams<WT> p) {
    pdl_launch();
    pdl_wait();
    const uint32_t t = blockIdx.x, pos = pos_of(p.ps) + t;
    uint32_t tok;
    if (p.ps.sp) { tok = p.ps.sp->token; if (threadIdx.x == 0) p.tokens[pos] = tok; }
    else tok = p.tokens[pos];
    const WT* e = p.embed + (size_t)tok * p.width;
    const WT* b = nullptr;
    if (p.bigram) {
        uint32_t row = p.buckets;
        if (pos > 0) {
            const uint32_t prev = p.tokens[pos - 1];
            row = (uint32_t)(((unsigned long long)prev * p.mul_prev + (unsigned long long)tok * p.mul_cur) % p.buckets);
        }
        b = p.bigram + (size_t)row * p.width;
    }
    float* x = p.x + (size_t)t * p.width;
    for (int c = threadIdx.x; c < p.width; c += blockDim.x) x[c] = to_f(e[c]) + (b ? to_f(b[c]) : 0.0f);
}

// ---- RMS norm of rows -----------------------------------------------------------------------------------------------
template <typename AT> struct NormRowsParams {
    const float* x; int ldx;
    const uint32_t* rows;   // optional gather: output row r reads input row rows[r]
    const float* w;         // may be null (unit norm)
    AT* out; int ldo;
    int n; float eps;
};
template <typename AT> __global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const NormRowsParams<AT> p) {
    __shared__ float red[33];
    pdl_launch();
    pdl_wait();
    const int r = blockIdx.x;
    const float* x = p.x + (size_t)(p.rows ? p.rows[r] : (uint32_t)r) * p.ldx;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < p.n; c += blockDim.x) { const float v = x[c]; ss += v * v; }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)p.n + p.eps);
    AT* o = p.out + (size_t)r * p.ldo;
    for (int c = threadIdx.x; c < p.n; c += blockDim.x) from_f(o[c], p.w ? x[c] * inv * p.w[c] : x[c] * inv);
}

// ---- norm without statistics: tanh(alpha * x) * w + b ------------------------------------------------------------------
struct TanhNorm {          // the three tensors of one such norm; alpha is one float on the device
    const float* alpha; const float* w; const float* b;
};
DN_DEVINL float tanhnorm_apply(const TanhNorm& n, float alpha, int c, float v) { return tanhf(alpha * v) * n.w[c] + n.b[c]; }
template <typename AT> struct TanhNormRowsParams {
    const float* x; int ldx;
    const uint32_t* rows;   // optional gather
    TanhNorm n;
    AT* out; int ldo;
    int width;
};
template <typename AT> __global__ void __launch_bounds__(256) tanhnorm_rows_kernel(const TanhNormRowsParams<AT> p) {
    pdl_launch();
    pdl_wait();
    const int r = blockIdx.x;
    const float* x = p.x + (size_t)(p.rows ? p.rows[r] : (uint32_t)r) * p.ldx;
    const float alpha = *p.n.alpha;
    AT* o = p.out + (size_t)r * p.ldo;
    for (int c = threadIdx.x; c < p.width; c += blockDim.x) from_f(o[c], tanhnorm_apply(p.n, alpha, c, x[c]));
}

// ---- layer norm without bias: (x - mean) / sqrt(mean((x - mean)^2) + eps) * w ---------------------------------------------
// v = LN(in row) * w.  With `resid`: v <- resid row + ls * v, written back to resid (a sublayer's normed output entering the
// residual stream).  v then goes to out_f (f32) and / or out_op (operand type: the input of the next matrix product).
template <typename AT> struct LayerNormRowsParams {
    const float* in; int ld_in;
    const uint32_t* rows;   // optional gather: output row r reads input row rows[r]
    const float* w; float eps; int n;
    float* resid; int ld_resid; const float* ls;
    float* out_f; int ld_f;
    AT* out_op; int ldo;
};
// mean and 1 / sqrt(var + eps) of n floats, two passes (the variance is the mean of the squared deviations)
DN_DEVINL void layernorm_stats(const float* x, int n, float* red, float& mean, float& inv, float eps) {
    float s = 0.0f;
    for (int c = threadIdx.x; c < n; c += blockDim.x) s += x[c];
    mean = block_sum(s, red) / (float)n;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < n; c += blockDim.x) { const float d = x[c] - mean; ss += d * d; }
    inv = 1.0f / sqrtf(block_sum(ss, red) / (float)n + eps);
}
// One row through the norm by a whole CTA: load(c) gives input column c (a plain read, or something computed); v = LN * w[c];
// with resid: v <- resid[c] + ls[c] * v, written back; v then goes to out_f and / or out_op.  The row is held in registers
// between the passes when it is short enough (n <= LN_CACHE * blockDim.x), so load runs once per column; longer rows load
// three times.
constexpr int LN_CACHE = 16;
template <typename AT, typename F>
DN_DEVINL void layernorm_row(F load, int n, const float* w, float eps, float* red, float* resid, const float* ls, float* out_f, AT* out_op) {
    const bool cached = n <= LN_CACHE * (int)blockDim.x;
    float v[LN_CACHE];
    float s = 0.0f;
    if (cached) {
#pragma unroll
        for (int i = 0; i < LN_CACHE; i++) {
            const int c = threadIdx.x + i * blockDim.x;
            v[i] = c < n ? load(c) : 0.0f;
            s += v[i];
        }
    } else {
        for (int c = threadIdx.x; c < n; c += blockDim.x) s += load(c);
    }
    const float mean = block_sum(s, red) / (float)n;
    float ss = 0.0f;
    if (cached) {
#pragma unroll
        for (int i = 0; i < LN_CACHE; i++) {
            const float d = threadIdx.x + i * blockDim.x < n ? v[i] - mean : 0.0f;
            ss += d * d;
        }
    } else {
        for (int c = threadIdx.x; c < n; c += blockDim.x) { const float d = load(c) - mean; ss += d * d; }
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)n + eps);
    auto finish = [&](int c, float in) {
        float o = (in - mean) * inv * w[c];
        if (resid) { o = resid[c] + ls[c] * o; resid[c] = o; }
        if (out_f) out_f[c] = o;
        if (out_op) from_f(out_op[c], o);
    };
    if (cached) {
#pragma unroll
        for (int i = 0; i < LN_CACHE; i++) {
            const int c = threadIdx.x + i * blockDim.x;
            if (c < n) finish(c, v[i]);
        }
    } else {
        for (int c = threadIdx.x; c < n; c += blockDim.x) finish(c, load(c));
    }
}
template <typename AT> __global__ void __launch_bounds__(256) layernorm_rows_kernel(const LayerNormRowsParams<AT> p) {
    __shared__ float red[33];
    pdl_launch();
    pdl_wait();
    const int r = blockIdx.x;
    const float* x = p.in + (size_t)(p.rows ? p.rows[r] : (uint32_t)r) * p.ld_in;
    layernorm_row<AT>([&](int c) { return x[c]; }, p.n, p.w, p.eps, red, p.resid ? p.resid + (size_t)r * p.ld_resid : nullptr, p.ls,
                      p.out_f ? p.out_f + (size_t)r * p.ld_f : nullptr, p.out_op ? p.out_op + (size_t)r * p.ldo : nullptr);
}

// ---- several residual streams -------------------------------------------------------------------------------------------
// Instead of one residual row a token carries S of them, X[0 .. S) (all equal to the embedding row at the start).  A sublayer
// reads u = sum_s win[s] X[s] (then normalised), and its output y is written to every stream at once from the old ones:
//     X'[t] = sum_s mix[s][t] X[s] + mult * wout[t] * y            (mix is indexed [from][to])
// One kernel does, per token, whatever of these is asked for, in this order: start the streams from `init`; apply the write
// of the sublayer that just ran; read for the next sublayer -- u (or the plain sum of the streams) stored in f32 and / or
// RMS-normalised with a weight and stored in the operand type.  A step of a layer is then one pass over the streams: the
// write of sublayer q and the read of sublayer q+1 share it.  One CTA per token (any block size up to 1024: a one-token step
// takes a large one); u stays in registers between the sum of squares and the output for rows up to STREAMS_CACHE * blockDim.x
// columns (longer rows recompute it from the streams just stored).
// S = 1 with win = wout = mix = 1 is the ordinary residual x <- x + mult * y.
constexpr int STREAMS_MAX = 16, STREAMS_CACHE = 8;
template <typename AT> struct StreamsParams {
    float* xs;                       // [T][S][width]
    int S, width;
    const float* init; int ld_init;  // or null
    const float* y; int ldy;         // or null: the sublayer output to write
    const float* mix; const float* wout; float mult;   // [S][S], [S]
    const float* win;                // or null: [S] read weights
    int sum_all;                     // 1: read the plain sum of the streams (win ignored)
    const uint32_t* rows;            // optional gather for a read-only pass: output row r reads token rows[r]
    float* u_out; int ldu;           // optional f32 copy of what was read
    const float* nw; float eps; AT* h; int ldh;   // optional: h = u / sqrt(mean(u^2) + eps) * nw
};
template <typename AT, int SMAX> __global__ void __launch_bounds__(1024) streams_step_kernel(const StreamsParams<AT> p) {
    __shared__ float red[33];
    __shared__ float cm[SMAX * SMAX], co[SMAX], ci[SMAX];
    pdl_launch();
    pdl_wait();
    const int r = blockIdx.x, S = p.S;
    const size_t t = p.rows ? p.rows[r] : (uint32_t)r;
    for (int i = threadIdx.x; i < SMAX * SMAX; i += blockDim.x) {
        const int s = i / SMAX, u = i % SMAX;
        cm[i] = (p.y && s < S && u < S) ? p.mix[s * S + u] : 0.0f;
    }
    for (int i = threadIdx.x; i < SMAX; i += blockDim.x) {
        co[i] = (p.y && i < S) ? p.mult * p.wout[i] : 0.0f;
        ci[i] = i < S ? (p.sum_all ? 1.0f : (p.win ? p.win[i] : 0.0f)) : 0.0f;
    }
    __syncthreads();
    float* X = p.xs + t * (size_t)S * p.width;
    auto read_u = [&](const float (&xv)[SMAX]) {
        float u = 0.0f;
#pragma unroll
        for (int s = 0; s < SMAX; s++) u = fmaf(ci[s], xv[s], u);
        return u;
    };
    // column c of every stream: load (or start from the embedding), ...
    auto load_col = [&](int c, float (&xv)[SMAX], float& yv) {
        if (p.init) {
            const float v = p.init[t * p.ld_init + c];
#pragma unroll
            for (int s = 0; s < SMAX; s++) xv[s] = s < S ? v : 0.0f;
        } else {
#pragma unroll
            for (int s = 0; s < SMAX; s++) xv[s] = s < S ? X[(size_t)s * p.width + c] : 0.0f;
        }
        yv = p.y ? p.y[t * p.ldy + c] : 0.0f;
    };
    // ... bring up to date, store, and return what the next sublayer reads there
    auto finish_col = [&](int c, float (&xv)[SMAX], float yv) {
        if (p.y) {
            float nx[SMAX];
#pragma unroll
            for (int u = 0; u < SMAX; u++) {
                float a = co[u] * yv;
#pragma unroll
                for (int s = 0; s < SMAX; s++) a = fmaf(cm[s * SMAX + u], xv[s], a);
                nx[u] = a;
            }
#pragma unroll
            for (int s = 0; s < SMAX; s++) xv[s] = nx[s];
        }
        if (p.y || p.init) {
#pragma unroll
            for (int s = 0; s < SMAX; s++)
                if (s < S) X[(size_t)s * p.width + c] = xv[s];
        }
        return read_u(xv);
    };
    auto column = [&](int c) {
        float xv[SMAX], yv;
        load_col(c, xv, yv);
        return finish_col(c, xv, yv);
    };
    const bool reads = p.win || p.sum_all;
    float uc[STREAMS_CACHE];
    float ss = 0.0f;
    // CB columns at a time: all their loads are issued before the first store (a store could alias a later load for all the
    // compiler knows, so column after column would wait for memory once per column)
    constexpr int CB = SMAX >= 16 ? 1 : (16 / SMAX > STREAMS_CACHE ? STREAMS_CACHE : 16 / SMAX);
#pragma unroll
    for (int i0 = 0; i0 < STREAMS_CACHE; i0 += CB) {
        float xv[CB][SMAX], yv[CB];
#pragma unroll
        for (int b = 0; b < CB; b++) {
            const int c = threadIdx.x + (i0 + b) * blockDim.x;
            if (c < p.width) load_col(c, xv[b], yv[b]);
        }
#pragma unroll
        for (int b = 0; b < CB; b++) {
            const int c = threadIdx.x + (i0 + b) * blockDim.x;
            uc[i0 + b] = c < p.width ? finish_col(c, xv[b], yv[b]) : 0.0f;
            ss = fmaf(uc[i0 + b], uc[i0 + b], ss);
            if (reads && p.u_out && c < p.width) p.u_out[(size_t)r * p.ldu + c] = uc[i0 + b];
        }
    }
    for (int c = threadIdx.x + STREAMS_CACHE * blockDim.x; c < p.width; c += blockDim.x) {
        const float u = column(c);
        ss = fmaf(u, u, ss);
        if (reads && p.u_out) p.u_out[(size_t)r * p.ldu + c] = u;
    }
    if (!reads || !p.h) return;
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)p.width + p.eps);
    AT* h = p.h + (size_t)r * p.ldh;
#pragma unroll
    for (int i = 0; i < STREAMS_CACHE; i++) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < p.width) from_f(h[c], uc[i] * inv * p.nw[c]);
    }
    for (int c = threadIdx.x + STREAMS_CACHE * blockDim.x; c < p.width; c += blockDim.x) {
        float xv[SMAX];
#pragma unroll
        for (int s = 0; s < SMAX; s++) xv[s] = s < S ? X[(size_t)s * p.width + c] : 0.0f;   // this thread stored them above
        from_f(h[c], read_u(xv) * inv * p.nw[c]);
    }
}

// ---- epilogues shared by the matrix kernels ---------------------------------------------------------------------------
enum { EPI_STORE = 0, EPI_RESID = 1, EPI_GLU = 2, EPI_ACT = 3 };
template <typename AT> struct EpiParams {
    float* out; int ldo;      // EPI_STORE: out = acc * scale (+ bias[o]);  EPI_RESID: out += ls[o] * f(acc) (+ lb[o])
    float scale;
    const float* ls;
    AT* act; int lda;         // EPI_GLU: act = glu(gate, up) in the operand type;  EPI_ACT: act = f(acc)
    const float* bias;        // EPI_STORE: optional bias of the projection
    const float* tanh_alpha;  // EPI_RESID: when set, f(acc) = tanh(*tanh_alpha * acc) (a tanh norm on the way into the residual)
    const float* lb;          // EPI_RESID: optional shift
    int glu_kind;             // EPI_GLU: GLU_SILU silu(gate) * up | GLU_CLAMPED g = min(gate, limit), u = clamp(up, +-limit):
    float glu_limit, glu_alpha;   //      g * sigmoid(glu_alpha * g) * (u + 1)
    int act_kind;             // EPI_ACT: ACT_NONE acc | ACT_RELU2 max(acc, 0)^2
};
enum { GLU_SILU = 0, GLU_CLAMPED = 1 };
enum { ACT_NONE = 0, ACT_RELU2 = 1 };
DN_DEVINL float silu(float z) { return z / (1.0f + expf(-z)); }
template <typename AT> DN_DEVINL float glu_apply(const EpiParams<AT>& e, float gate, float up) {
    if (e.glu_kind == GLU_CLAMPED) {
        const float g = fminf(gate, e.glu_limit), u = fminf(fmaxf(up, -e.glu_limit), e.glu_limit);
        return g / (1.0f + expf(-e.glu_alpha * g)) * (u + 1.0f);
    }
    return silu(gate) * up;
}
template <typename AT> DN_DEVINL float act_apply(const EpiParams<AT>& e, float a) {
    if (e.act_kind == ACT_RELU2) { const float r = fmaxf(a, 0.0f); return r * r; }
    return a;
}
template <int EPI, typename AT> DN_DEVINL void epi_apply(const EpiParams<AT>& e, int t, int o, float a, float b) {
    if (EPI == EPI_STORE) e.out[(size_t)t * e.ldo + o] = e.bias ? a * e.scale + e.bias[o] : a * e.scale;
    else if (EPI == EPI_RESID) {
        if (e.tanh_alpha) a = tanhf(*e.tanh_alpha * a);
        e.out[(size_t)t * e.ldo + o] += e.lb ? e.ls[o] * a + e.lb[o] : e.ls[o] * a;
    }
    else if (EPI == EPI_GLU) from_f(e.act[(size_t)t * e.lda + o], glu_apply(e, a, b));
    else from_f(e.act[(size_t)t * e.lda + o], act_apply(e, a));
}

// ---- one row times a matrix: W [O][K] streamed once ----------------------------------------------------------------------
// A warp owns output rows o = warp, warp + nwarps, ...; lanes walk K in 16-byte pieces, four pieces in flight per lane.
// NORM: the input row is the f32 residual, normalised here and rounded to the operand type exactly as the row kernels
// (rmsnorm_rows_kernel, tanhnorm_rows_kernel) do, so both routes feed the product the same numbers.
//   NORM_RMS   x * rsqrt(mean x^2 + eps) * nw          NORM_TANH   tanh(alpha x) w + b
//   NORM_LAYER (x - mean) * rsqrt(var + eps) * nw
// Batch (gridDim.y > 1): CTA row y multiplies input a + y * a_bs by matrix w + bidx[y] * w_bs (bidx null: y itself) and
// writes at out/act + y * o_bs -- one matrix per head, or the experts a router picked, read from its device-side list.  A
// list entry >= n_mats (when n_mats > 0) names an expert without matrices: its CTAs leave at once.
enum { NORM_NONE = 0, NORM_RMS = 1, NORM_TANH = 2, NORM_LAYER = 3 };
// What follows an EPI_STORE product whose whole output row is a sublayer's result (ln.counter set): the CTA that finishes last
// -- every CTA takes a ticket from *counter after its stores -- sends the row e.out[0 .. O) through a layer norm into the
// residual stream, x <- x + ls * LN(row) w, and writes x again in the operand type to h.  Nobody waits for anybody: the last
// ticket simply falls to whoever comes last, and that CTA puts the counter back to zero.
template <typename AT> struct LnTail {
    unsigned int* counter;
    const float* w; const float* ls; float eps;
    float* x; AT* h;
};
template <typename AT, typename WT> struct GemvRowsParams {
    const AT* a;              // [K] input row (NORM_NONE)
    const float* x; const float* nw; float eps;   // NORM_RMS, NORM_LAYER
    TanhNorm tn;                                  // NORM_TANH
    const WT* w; const WT* w2;   // [O][K]; w2: the "up" matrix of EPI_GLU
    int K, O;
    int ksplit;               // 1: the warps of a CTA split K of one row pair (few rows), 0: a warp per row pair
    int pdl;                  // launched with programmatic dependent launch: prefetch weights before waiting for the input
    EpiParams<AT> e;
    const int* bidx; long long a_bs, w_bs, o_bs;
    int n_mats;
    LnTail<AT> ln;
};
template <typename WT> struct Vec16;
template <> struct Vec16<float> { static constexpr int N = 4; };
template <> struct Vec16<__nv_bfloat16> { static constexpr int N = 8; };
template <typename WT> DN_DEVINL void load16(const WT* p, float (&v)[Vec16<WT>::N]);
template <> DN_DEVINL void load16<float>(const float* p, float (&v)[4]) {
    const float4 q = __ldcs(reinterpret_cast<const float4*>(p));
    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
}
template <> DN_DEVINL void load16<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 q = __ldcs(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; i++) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}
// NR weight rows against the same input row: the shared-memory reads of the input are paid once for NR rows
template <typename WT, int NR>
DN_DEVINL void dot_rows(const WT* const (&w)[NR], const float* __restrict__ xs, int K, int lane, bool vec, float (&out)[NR]) {
    constexpr int N = Vec16<WT>::N;
    float acc[NR];
#pragma unroll
    for (int r = 0; r < NR; r++) acc[r] = 0.0f;
    if (vec) {
        const int pieces = K / N;
        int i = lane;
        for (; i + 32 < pieces; i += 64) {
            float v[NR][2][N];
#pragma unroll
            for (int r = 0; r < NR; r++) { load16<WT>(w[r] + (size_t)i * N, v[r][0]); load16<WT>(w[r] + (size_t)(i + 32) * N, v[r][1]); }
#pragma unroll
            for (int u = 0; u < 2; u++) {
                float xv[N];
#pragma unroll
                for (int j = 0; j < N; j += 4) {
                    const float4 x4 = *reinterpret_cast<const float4*>(xs + (size_t)(i + 32 * u) * N + j);
                    xv[j] = x4.x; xv[j + 1] = x4.y; xv[j + 2] = x4.z; xv[j + 3] = x4.w;
                }
#pragma unroll
                for (int r = 0; r < NR; r++)
#pragma unroll
                    for (int j = 0; j < N; j++) acc[r] = fmaf(v[r][u][j], xv[j], acc[r]);
            }
        }
        for (; i < pieces; i += 32) {
            float xv[N];
#pragma unroll
            for (int j = 0; j < N; j += 4) {
                const float4 x4 = *reinterpret_cast<const float4*>(xs + (size_t)i * N + j);
                xv[j] = x4.x; xv[j + 1] = x4.y; xv[j + 2] = x4.z; xv[j + 3] = x4.w;
            }
#pragma unroll
            for (int r = 0; r < NR; r++) {
                float v0[N];
                load16<WT>(w[r] + (size_t)i * N, v0);
#pragma unroll
                for (int j = 0; j < N; j++) acc[r] = fmaf(v0[j], xv[j], acc[r]);
            }
        }
    } else {
        for (int k = lane; k < K; k += 32)
#pragma unroll
            for (int r = 0; r < NR; r++) acc[r] = fmaf(to_f(w[r][k]), xs[k], acc[r]);
    }
#pragma unroll
    for (int r = 0; r < NR; r++) out[r] = warp_sum(acc[r]);
}
template <typename AT, typename WT, int EPI, int NORM>
static __global__ void __launch_bounds__(256) gemv_rows_kernel(const GemvRowsParams<AT, WT> pp) {
    extern __shared__ __align__(16) float gv_xs[];   // [K rounded up to 4] the input row as f32, then reduction slots
    GemvRowsParams<AT, WT> p = pp;
    float* red = gv_xs + ((p.K + 3) & ~3);
    pdl_launch();
    if (gridDim.y > 1 || p.bidx) {   // the expert list is written by the step's router kernel: read it after the wait
        if (p.bidx) pdl_wait();
        const long long by = blockIdx.y, bw = p.bidx ? p.bidx[by] : by;
        if (p.n_mats > 0 && bw >= p.n_mats) return;
        p.w += bw * p.w_bs;
        if (p.w2) p.w2 += bw * p.w_bs;
        if (p.a) p.a += by * p.a_bs;
        if (p.e.out) p.e.out += by * p.o_bs;
        if (p.e.act) p.e.act += by * p.o_bs;
    }
    if (p.pdl) {   // weights do not depend on the predecessor: ask L2 for this warp's first rows while waiting for it
        const int w0 = (int)(blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5));
        const int o = p.ksplit ? 2 * (int)blockIdx.x : (EPI == EPI_GLU ? w0 : 2 * w0);
        if (o < p.O) {
            const char* base = reinterpret_cast<const char*>(p.w + (size_t)o * p.K);
            const size_t bytes = (size_t)p.K * sizeof(WT) * (EPI == EPI_GLU ? 1 : (o + 1 < p.O ? 2 : 1));
            const size_t lo = p.ksplit ? bytes * (threadIdx.x >> 5) / (blockDim.x >> 5) : 0;
            const size_t hi = p.ksplit ? bytes * ((threadIdx.x >> 5) + 1) / (blockDim.x >> 5) : bytes;
            for (size_t b = lo + (size_t)(threadIdx.x & 31) * 128; b < hi && b < lo + 8192; b += 32 * 128)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(base + b));
            if (EPI == EPI_GLU) {
                const char* base2 = reinterpret_cast<const char*>(p.w2 + (size_t)o * p.K);
                for (size_t b = (size_t)(threadIdx.x & 31) * 128; b < bytes && b < 8192; b += 32 * 128)
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(base2 + b));
            }
        }
    }
    pdl_wait();
    if (NORM == NORM_RMS) {
        float ss = 0.0f;
        for (int c = threadIdx.x; c < p.K; c += blockDim.x) { const float v = p.x[c]; ss += v * v; }
        ss = block_sum(ss, red);
        const float inv = 1.0f / sqrtf(ss / (float)p.K + p.eps);
        for (int c = threadIdx.x; c < p.K; c += blockDim.x) { AT r; from_f(r, p.x[c] * inv * p.nw[c]); gv_xs[c] = to_f(r); }
    } else if (NORM == NORM_LAYER) {
        float mean, inv;
        layernorm_stats(p.x, p.K, red, mean, inv, p.eps);
        for (int c = threadIdx.x; c < p.K; c += blockDim.x) { AT r; from_f(r, (p.x[c] - mean) * inv * p.nw[c]); gv_xs[c] = to_f(r); }
    } else if (NORM == NORM_TANH) {
        const float alpha = *p.tn.alpha;
        for (int c = threadIdx.x; c < p.K; c += blockDim.x) { AT r; from_f(r, tanhnorm_apply(p.tn, alpha, c, p.x[c])); gv_xs[c] = to_f(r); }
    } else {
        for (int c = threadIdx.x; c < p.K; c += blockDim.x) gv_xs[c] = to_f(p.a[c]);
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const bool vec = p.K % Vec16<WT>::N == 0;   // every weight row then starts on a 16-byte boundary
    if (p.ksplit) {
        // few output rows (a down or output projection): a warp per row pair would leave most of the GPU idle, so the
        // warps of a CTA share a row pair, each walking one slice of K; partial sums meet in shared memory
        constexpr int N = Vec16<WT>::N;
        const int pieces = p.K / N;                                // ksplit is only chosen when K % N == 0
        const int per = (pieces + nw - 1) / nw;
        const int k0 = min(pieces, warp * per) * N, k1 = min(pieces, (warp + 1) * per) * N;
        float* part = red + 36;                                    // [2][nw]
        for (int o = 2 * blockIdx.x; o < p.O; o += 2 * gridDim.x) {
            const int o1 = o + 1 < p.O ? o + 1 : o;
            const WT* const rows[2] = {p.w + (size_t)o * p.K + k0, p.w + (size_t)o1 * p.K + k0};
            float r[2];
            dot_rows<WT, 2>(rows, gv_xs + k0, k1 - k0, lane, true, r);
            if (lane == 0) { part[warp] = r[0]; part[nw + warp] = r[1]; }
            __syncthreads();
            if (warp == 0 && lane < 2) {
                float a = 0.0f;
                for (int w = 0; w < nw; w++) a += part[lane * nw + w];
                if (lane == 0) epi_apply<EPI, AT>(p.e, 0, o, a, 0.0f);
                else if (o1 != o) epi_apply<EPI, AT>(p.e, 0, o1, a, 0.0f);
            }
            __syncthreads();
        }
    } else if (EPI == EPI_GLU) {
        for (int o = blockIdx.x * nw + warp; o < p.O; o += gridDim.x * nw) {
            const WT* const rows[2] = {p.w + (size_t)o * p.K, p.w2 + (size_t)o * p.K};
            float r[2];
            dot_rows<WT, 2>(rows, gv_xs, p.K, lane, vec, r);
            if (lane == 0) epi_apply<EPI, AT>(p.e, 0, o, r[0], r[1]);
        }
    } else {
        for (int o = 2 * (blockIdx.x * nw + warp); o < p.O; o += 2 * gridDim.x * nw) {
            const int o1 = o + 1 < p.O ? o + 1 : o;
            const WT* const rows[2] = {p.w + (size_t)o * p.K, p.w + (size_t)o1 * p.K};
            float r[2];
            dot_rows<WT, 2>(rows, gv_xs, p.K, lane, vec, r);
            if (lane == 0) {
                epi_apply<EPI, AT>(p.e, 0, o, r[0], 0.0f);
                if (o1 != o) epi_apply<EPI, AT>(p.e, 0, o1, r[1], 0.0f);
            }
        }
    }
    if (EPI == EPI_STORE && p.ln.counter) {
        __shared__ unsigned int last;
        __threadfence();   // this thread's stores of the row before the ticket
        __syncthreads();
        if (threadIdx.x == 0) {
            const unsigned int ticket = atomicAdd(p.ln.counter, 1u);
            last = ticket == gridDim.x * gridDim.y - 1 ? 1u : 0u;
        }
        __syncthreads();
        if (last) {
            __threadfence();
            const float* row = p.e.out;
            layernorm_row<AT>([&](int c) { return __ldcg(row + c); }, p.O, p.ln.w, p.ln.eps, red, p.ln.x, p.ln.ls, nullptr, p.ln.h);
            if (threadIdx.x == 0) *p.ln.counter = 0u;
        }
    }
}

// ---- many rows times a matrix on CUDA cores: out[T][O] = A[T][K] . W[O][K]^T, any shape --------------------------------
// 64 x 64 output tile, K in steps of 16, 256 threads x (4 x 4) outputs; each output element adds its products in
// ascending k, so a row's result does not depend on how many rows the call has.
// blockIdx.z = batch entry z: matrix w + z * w_bs; without `grp` the input columns start at a + z * a_bs and the output
// columns at out/act + z * o_bs (one matrix per head); with `grp` (device, [batches + 1] ascending row offsets) entry z owns
// rows grp[z] .. grp[z+1] of the input and the output (one matrix per expert over rows sorted by expert).
template <typename AT, typename WT> struct GemmTiledParams {
    const AT* a; int lda;
    const WT* w; const WT* w2;
    int T, K, O;
    EpiParams<AT> e;
    const int* grp; long long a_bs, w_bs, o_bs;
};
template <typename AT, typename WT, int EPI>
static __global__ void __launch_bounds__(256) gemm_tiled_kernel(const GemmTiledParams<AT, WT> pp) {
    constexpr int BM = 64, BN = 64, BK = 16;
    constexpr bool GLU = EPI == EPI_GLU;
    pdl_launch();
    pdl_wait();
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    __shared__ float W2s[GLU ? BK : 1][BN + 4];
    GemmTiledParams<AT, WT> p = pp;
    int row0 = 0;
    if (gridDim.z > 1 || p.grp) {
        const long long z = blockIdx.z;
        p.w += z * p.w_bs;
        if (p.w2) p.w2 += z * p.w_bs;
        if (p.grp) { row0 = p.grp[z]; p.T = p.grp[z + 1]; }
        else { p.a += z * p.a_bs; if (p.e.out) p.e.out += z * p.o_bs; if (p.e.act) p.e.act += z * p.o_bs; }
    }
    const int m0 = row0 + blockIdx.y * BM, n0 = blockIdx.x * BN;
    if (m0 >= p.T) return;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4] = {}, acc2[GLU ? 4 : 1][4] = {};
    const int lr = threadIdx.x >> 2, lk = (threadIdx.x & 3) * 4;   // loader: row lr of the tile, k offset lk .. lk+3
    for (int k0 = 0; k0 < p.K; k0 += BK) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int k = k0 + lk + j;
            As[lk + j][lr] = (m0 + lr < p.T && k < p.K) ? to_f(p.a[(size_t)(m0 + lr) * p.lda + k]) : 0.0f;
            Ws[lk + j][lr] = (n0 + lr < p.O && k < p.K) ? to_f(p.w[(size_t)(n0 + lr) * p.K + k]) : 0.0f;
            if (GLU) W2s[lk + j][lr] = (n0 + lr < p.O && k < p.K) ? to_f(p.w2[(size_t)(n0 + lr) * p.K + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; k++) {
            const float4 a4 = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
            const float4 w4 = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
            const float av[4] = {a4.x, a4.y, a4.z, a4.w}, wv[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
            if (GLU) {
                const float4 u4 = *reinterpret_cast<const float4*>(&W2s[k][tx * 4]);
                const float uv[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int j = 0; j < 4; j++) acc2[GLU ? i : 0][j] = fmaf(av[i], uv[j], acc2[GLU ? i : 0][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int t = m0 + ty * 4 + i, o = n0 + tx * 4 + j;
            if (t < p.T && o < p.O) epi_apply<EPI, AT>(p.e, t, o, acc[i][j], acc2[GLU ? i : 0][j]);
        }
}

// ---- what happens to q, k, v (and the gate logits) between the projection and the attention ---------------------------
// Input: one row per token of the fused projection [q (H*dk) | k (G*dk) | v (G*dv) | gate logits (H, optional)], f32.
//   qk_mode QK_UNITNORM: every q and k head is divided by its root mean square (eps inside the root), no weight
//   qk_mode QK_ROTARY:   the first rot_dims dimensions of every q and k head are rotated, dimension i paired with
//                        i + rot_dims/2, by the angle position * f_i taken from host-made cos/sin tables [pos][rot_dims/2]
//   q_nw / k_nw:         when set, every q (k) head is first RMS-normalised (eps inside the root) and multiplied by this
//                        weight [dk], the same for all heads; QK_ROTARY or QK_PLAIN then act on the normalised head
//   v_mode  V_FIRST:     the values are also kept in v_first (this step's rows) for later layers
//   v_mode  V_MIX:       v <- (1 - lambda) v + lambda v_first
// q goes to q_out [T][H*dk], k and v to cache rows pos+t, sigmoid(gate logit) to gate_out [T][H].
enum { QK_PLAIN = 0, QK_UNITNORM = 1, QK_ROTARY = 2 };
enum { V_PLAIN = 0, V_FIRST = 1, V_MIX = 2 };
struct QkvPostParams {
    const float* qkv; int ld;
    int H, G, dk, dv;
    int qk_mode; float eps;
    const float* q_nw; const float* k_nw;                       // [dk] or null
    int rot_dims; const float* rot_cos; const float* rot_sin;   // [max_tokens][rot_dims/2]
    int v_mode; float* v_first; const float* lambda;            // v_first [T][G*dv]; lambda: one float on the device
    bool has_gate;
    float* q_out; float* gate_out;
    float* kcache; float* vcache;                               // [max_tokens][G*dk], [max_tokens][G*dv]
    PosSrc ps;
};
static __global__ void __launch_bounds__(128) qkv_post_kernel(const QkvPostParams p) {
    // grid (T, Y): the warps of the Y CTAs of a token share its tasks -- one per q head, one per k head, one per 128
    // value elements, one for the gates
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    const uint32_t pos = pos_of(p.ps) + (uint32_t)t;
    const int lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int wid = blockIdx.y * nw + (threadIdx.x >> 5), wtotal = gridDim.y * nw;
    const float* row = p.qkv + (size_t)t * p.ld;
    const int n_qk = p.H + p.G, nv = p.G * p.dv, v_tasks = (nv + 127) / 128;
    const float* vsrc = row + (size_t)n_qk * p.dk;
    const int n_tasks = n_qk + v_tasks + (p.has_gate ? 1 : 0);
    for (int task = wid; task < n_tasks; task += wtotal) {
        if (task >= n_qk + v_tasks) {
            for (int h = lane; h < p.H; h += 32) p.gate_out[(size_t)t * p.H + h] = 1.0f / (1.0f + expf(-vsrc[nv + h]));
            continue;
        }
        if (task >= n_qk) {
            const float lam = p.v_mode == V_MIX ? *p.lambda : 0.0f;
            const int i1 = min(nv, (task - n_qk + 1) * 128);
            for (int i = (task - n_qk) * 128 + lane; i < i1; i += 32) {
                float v = vsrc[i];
                if (p.v_mode == V_FIRST) p.v_first[(size_t)t * nv + i] = v;
                else if (p.v_mode == V_MIX) v = (1.0f - lam) * v + lam * p.v_first[(size_t)t * nv + i];
                p.vcache[(size_t)pos * nv + i] = v;
            }
            continue;
        }
        const bool is_q = task < p.H;
        const float* src = row + (size_t)task * p.dk;  // k heads follow the q heads directly
        float* dst = is_q ? p.q_out + ((size_t)t * p.H + task) * p.dk : p.kcache + ((size_t)pos * p.G + (task - p.H)) * p.dk;
        if (p.qk_mode == QK_UNITNORM) {
            float ss = 0.0f;
            for (int d = lane; d < p.dk; d += 32) ss += src[d] * src[d];
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)p.dk + p.eps);
            for (int d = lane; d < p.dk; d += 32) dst[d] = src[d] * inv;
        } else {
            const float* nw = is_q ? p.q_nw : p.k_nw;
            float inv = 1.0f;
            if (nw) {
                float ss = 0.0f;
                for (int d = lane; d < p.dk; d += 32) ss += src[d] * src[d];
                ss = warp_sum(ss);
                inv = 1.0f / sqrtf(ss / (float)p.dk + p.eps);
            }
            auto val = [&](int d) { return nw ? src[d] * inv * nw[d] : src[d]; };
            const int rot = p.qk_mode == QK_ROTARY ? p.rot_dims : 0, half = rot / 2;
            const float* c = p.rot_cos + (size_t)pos * half;
            const float* s = p.rot_sin + (size_t)pos * half;
            for (int i = lane; i < half; i += 32) {
                const float u = val(i), v = val(i + half);
                dst[i] = u * c[i] - v * s[i];
                dst[i + half] = v * c[i] + u * s[i];
            }
            for (int d = rot + lane; d < p.dk; d += 32) dst[d] = val(d);
        }
    }
}

// ---- attention --------------------------------------------------------------------------------------------------------
// score = (q . k) * scale, then softcap * tanh(score / softcap) when softcap > 0, then minus r1[head] * ln(1 + r2[head] *
// distance) when r1 is given; row (t, head) at position i = pos+t sees keys j <= i, and only those with i - j < window or
// j < keep_first when window > 0 (key tiles wholly between the kept first keys and the window are never loaded); softmax in
// f32, its denominator enlarged by exp(sink[head]) when a sink is given; output row times the head's gate or times
// per-element sigmoid gates (when given), written in the operand type as [T][H*dv].
// CTA = (tile of TQ query tokens, KV head, chunk of HC query heads of that KV head[, key split]); 4 warps x RW row slots,
// row slot r = (token r / HC, head r % HC).  Keys are walked in tiles of 64 staged in shared memory: lane j scores keys j
// and j + 32 of the tile for each of its rows (K rows padded so that the 16-byte reads of 32 lanes do not collide), an
// online softmax keeps (max, sum) per row, the probabilities go through shared memory and lane c accumulates output
// columns c, c + 32, ... .  Tiles start at multiples of 64 keys whatever the portion, so a row's arithmetic does not
// depend on how the prompt was cut.  With nsplit > 1 (decode) CTA `split` walks tiles split, split + nsplit, ... and writes
// (max, sum, unnormalised row) to scratch for attn_combine_kernel.
constexpr int ATT_KT = 64, ATT_WARPS = 4;
// exp and tanh of the attention inner loop on the special-function unit: ex2.approx is good to about 2e-7 relative, and
// cap * (1 - 2 / (e^(2s/cap) + 1)) then carries an absolute error of about cap * 1e-7 -- the size of the f32 rounding of the
// score itself (a relative error near zero does not matter: what enters the softmax is the score's absolute value)
DN_DEVINL float att_exp(float x) { return __expf(x); }
DN_DEVINL float att_softcap(float s, float cap, float inv_cap2) {   // inv_cap2 = 2 / cap
    return cap * (1.0f - __fdividef(2.0f, __expf(s * inv_cap2) + 1.0f));
}
template <typename AT> struct AttnRowsParams {
    const float* q;           // [T][H*dk]
    const float* kcache; const float* vcache;
    const float* gate;        // [T][H] or null
    AT* out;                  // [T][H*dv]
    float* part;              // nsplit > 1: [T][H][nsplit][dv + 2]
    int T, H, G, dk, dv, TQ, HC, nsplit;
    int k_ld, v_ld;           // floats between consecutive positions of the K and of the V cache (>= G*dk, G*dv)
    int window;               // > 0: sliding window of that many keys (the row's own included); 0: all earlier keys
    int keep_first;           // with a window: keys at positions < keep_first stay visible to every later row
    const float* sink;        // [H] or null: exp(sink[head]) is added to the softmax denominator (no key, no value, not scaled)
    const float* gate_logits; int gate_ld;   // or null: output element (t, h, c) is multiplied by sigmoid(gate_logits[t*gate_ld + h*dv + c])
    const float* r1; const float* r2;   // [H] distance penalty r1 * ln(1 + r2 * (i - j)), or null
    int nbuf;                 // 2: K/V tiles double-buffered with cp.async (needs dk % 4 == 0 and dv % 4 == 0), 1: loaded in place
    float scale, softcap;
    int out_ld;               // operand-type elements between consecutive tokens of `out` (H*dv unless the heads are written into a wider row)
    int has_out_scale;        // 1: the output row times out_scale (a mixer that is summed with another one at a fixed weight)
    float out_scale;
    PosSrc ps;
};
DN_DEVINL void cp_async16_zfill(void* smem_dst, const void* gsrc, bool valid) {   // 16 bytes, zeros when !valid
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(n) : "memory");
}
inline int attn_k_stride(int dk) { const int d4 = (dk + 3) & ~3; return d4 + ((4 - d4 % 32) + 32) % 32; }   // == 4 mod 32
template <int RW, int NI> inline size_t attn_smem_bytes(int dk, int dv, int nbuf) {
    const int d4 = (dk + 3) & ~3, R = RW * ATT_WARPS;
    return ((size_t)R * d4 + (size_t)nbuf * ((size_t)ATT_KT * attn_k_stride(dk) + (size_t)ATT_KT * 32 * NI) + (size_t)R * ATT_KT) * 4;
}
template <typename AT, int RW, int NI>
static __global__ void __launch_bounds__(ATT_WARPS * 32) attn_rows_kernel(const AttnRowsParams<AT> p) {
    constexpr int R = RW * ATT_WARPS, DVP = 32 * NI;
    pdl_launch();
    pdl_wait();
    extern __shared__ float at_sm[];
    const int d4 = (p.dk + 3) & ~3, ks = d4 + ((4 - d4 % 32) + 32) % 32;
    float* Qs = at_sm;                                  // [R][d4]
    float* Ks0 = Qs + (size_t)R * d4;                   // [nbuf][64][ks]
    float* Vs0 = Ks0 + (size_t)p.nbuf * ATT_KT * ks;    // [nbuf][64][DVP]
    float* Ps = Vs0 + (size_t)p.nbuf * ATT_KT * DVP;    // [R][64]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int kv_mul = p.H / p.G;
    const int chunks = (kv_mul + p.HC - 1) / p.HC;
    const int g = blockIdx.y / chunks, h0 = (blockIdx.y % chunks) * p.HC;
    const int t0 = (int)(gridDim.x - 1 - blockIdx.x) * p.TQ;   // late query tiles see the most keys: they are scheduled first
    const int split = blockIdx.z;
    const uint32_t pos0 = pos_of(p.ps);
    // row slots
    int r_t[RW], r_h[RW];
    bool r_ok[RW];
#pragma unroll
    for (int i = 0; i < RW; i++) {
        const int r = warp * RW + i;
        r_t[i] = t0 + r / p.HC;
        const int hl = h0 + r % p.HC;
        r_h[i] = g * kv_mul + hl;
        r_ok[i] = r / p.HC < p.TQ && r_t[i] < p.T && hl < kv_mul;
    }
    for (int e = threadIdx.x; e < R * d4; e += blockDim.x) {
        const int r = e / d4, d = e - r * d4;
        const int t = t0 + r / p.HC, hl = h0 + r % p.HC;
        const bool ok = r / p.HC < p.TQ && t < p.T && hl < kv_mul && d < p.dk;
        Qs[e] = ok ? p.q[((size_t)t * p.H + g * kv_mul + hl) * p.dk + d] : 0.0f;
    }
    const int t_last = min(p.T, t0 + p.TQ) - 1;
    const int n_keys = (int)pos0 + t_last + 1;           // keys this CTA's last row sees
    const int n_tiles = (n_keys + ATT_KT - 1) / ATT_KT;
    // the CTA's first row has the earliest window: tiles before its first visible key are skipped by every row
    const int first_tile = p.window > 0 ? max(0, (int)pos0 + t0 - p.window + 1) / ATT_KT : 0;
    // ... except the tiles of the kept first keys: the walk is tiles 0 .. kf_tiles, then first_tile .. n_tiles
    const int kf_tiles = p.window > 0 && p.keep_first > 0 ? min(first_tile, (p.keep_first + ATT_KT - 1) / ATT_KT) : 0;
    const int n_walk = kf_tiles + n_tiles - first_tile;
    auto tile_of = [&](int u) { return u < kf_tiles ? u : first_tile + (u - kf_tiles); };
    float m[RW], l[RW], acc[RW][NI];
    float pen1[RW], pen2[RW];
#pragma unroll
    for (int i = 0; i < RW; i++) { pen1[i] = p.r1 && r_ok[i] ? p.r1[r_h[i]] : 0.0f; pen2[i] = p.r1 && r_ok[i] ? p.r2[r_h[i]] : 0.0f; }
#pragma unroll
    for (int i = 0; i < RW; i++) {
        // the sink enters like a key with score sink[head] and no value; with split keys it belongs to split 0
        const bool sk = p.sink && r_ok[i] && blockIdx.z == 0;
        m[i] = sk ? p.sink[r_h[i]] : -1e30f; l[i] = sk ? 1.0f : 0.0f;
#pragma unroll
        for (int c = 0; c < NI; c++) acc[i][c] = 0.0f;
    }
    const size_t krow = (size_t)p.k_ld, vrow = (size_t)p.v_ld;
    const bool vec4 = (p.dk & 3) == 0 && (p.dv & 3) == 0 && (p.k_ld & 3) == 0 && (p.v_ld & 3) == 0;
    const bool async = p.nbuf == 2;
    const float inv_cap2 = p.softcap > 0.0f ? 2.0f / p.softcap : 0.0f;
    // double-buffered form: the copies of tile i+1 are in flight (cp.async, no registers) while tile i is used
    auto issue_tile = [&](int tile, int buf) {
        const int j0 = tile * ATT_KT;
        float* Kb = Ks0 + (size_t)buf * ATT_KT * ks;
        float* Vb = Vs0 + (size_t)buf * ATT_KT * DVP;
        const int kq = p.dk >> 2, vq = p.dv >> 2;
        for (int e = threadIdx.x; e < ATT_KT * kq; e += blockDim.x) {
            const int j = e / kq, d = (e - j * kq) << 2;
            const bool ok = j0 + j < n_keys;
            cp_async16_zfill(Kb + j * ks + d, ok ? p.kcache + (size_t)(j0 + j) * krow + (size_t)g * p.dk + d : p.kcache, ok);
        }
        for (int e = threadIdx.x; e < ATT_KT * vq; e += blockDim.x) {
            const int j = e / vq, c = (e - j * vq) << 2;
            const bool ok = j0 + j < n_keys;
            cp_async16_zfill(Vb + j * DVP + c, ok ? p.vcache + (size_t)(j0 + j) * vrow + (size_t)g * p.dv + c : p.vcache, ok);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (async) {
        if (p.dv < DVP)   // value columns beyond vdim are read by the p.V loop: zero them once in both buffers
            for (int e = threadIdx.x; e < 2 * ATT_KT * (DVP - p.dv); e += blockDim.x) {
                const int j = e / (DVP - p.dv), c = p.dv + (e - j * (DVP - p.dv));
                Vs0[(size_t)j * DVP + c] = 0.0f;
            }
        if (split < n_walk) issue_tile(tile_of(split), 0);
    }
    int buf = 0;
    for (int u = split; u < n_walk; u += p.nsplit) {
        const int tile = tile_of(u);
        const int j0 = tile * ATT_KT;
        float* Ks = Ks0 + (size_t)buf * ATT_KT * ks;
        float* Vs = Vs0 + (size_t)buf * ATT_KT * DVP;
        if (async) {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncthreads();   // this tile has landed for everyone, and everyone is done with the other buffer
            if (u + p.nsplit < n_walk) issue_tile(tile_of(u + p.nsplit), buf ^ 1);
            buf ^= 1;
        } else {
        __syncthreads();   // previous tile fully consumed (also orders the Qs fill before the first use)
        if (vec4) {   // head sizes in whole 16-byte pieces: every K and V row of this head starts on a 16-byte boundary
            const int kq = d4 >> 2;
            for (int e = threadIdx.x; e < ATT_KT * kq; e += blockDim.x) {
                const int j = e / kq, d = (e - j * kq) << 2;
                float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (j0 + j < n_keys) v = *reinterpret_cast<const float4*>(p.kcache + (size_t)(j0 + j) * krow + (size_t)g * p.dk + d);
                *reinterpret_cast<float4*>(Ks + j * ks + d) = v;
            }
            constexpr int VQ = DVP >> 2;
            for (int e = threadIdx.x; e < ATT_KT * VQ; e += blockDim.x) {
                const int j = e / VQ, c = (e - j * VQ) << 2;
                float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (j0 + j < n_keys && c < p.dv) v = *reinterpret_cast<const float4*>(p.vcache + (size_t)(j0 + j) * vrow + (size_t)g * p.dv + c);
                *reinterpret_cast<float4*>(Vs + j * DVP + c) = v;
            }
        } else {
            for (int e = threadIdx.x; e < ATT_KT * d4; e += blockDim.x) {
                const int j = e / d4, d = e - j * d4;
                Ks[j * ks + d] = (j0 + j < n_keys && d < p.dk) ? p.kcache[(size_t)(j0 + j) * krow + (size_t)g * p.dk + d] : 0.0f;
            }
            for (int e = threadIdx.x; e < ATT_KT * DVP; e += blockDim.x) {
                const int j = e / DVP, c = e - j * DVP;
                Vs[e] = (j0 + j < n_keys && c < p.dv) ? p.vcache[(size_t)(j0 + j) * vrow + (size_t)g * p.dv + c] : 0.0f;
            }
        }
        __syncthreads();
        }
        float s0[RW], s1[RW];
#pragma unroll
        for (int i = 0; i < RW; i++) { s0[i] = 0.0f; s1[i] = 0.0f; }
        const float* k0p = Ks + (size_t)lane * ks;
        const float* k1p = Ks + (size_t)(lane + 32) * ks;
        for (int d = 0; d < d4; d += 4) {
            const float4 ka = *reinterpret_cast<const float4*>(k0p + d);
            const float4 kb = *reinterpret_cast<const float4*>(k1p + d);
#pragma unroll
            for (int i = 0; i < RW; i++) {
                const float4 qv = *reinterpret_cast<const float4*>(Qs + (size_t)(warp * RW + i) * d4 + d);
                s0[i] = fmaf(qv.x, ka.x, s0[i]); s0[i] = fmaf(qv.y, ka.y, s0[i]); s0[i] = fmaf(qv.z, ka.z, s0[i]); s0[i] = fmaf(qv.w, ka.w, s0[i]);
                s1[i] = fmaf(qv.x, kb.x, s1[i]); s1[i] = fmaf(qv.y, kb.y, s1[i]); s1[i] = fmaf(qv.z, kb.z, s1[i]); s1[i] = fmaf(qv.w, kb.w, s1[i]);
            }
        }
        float corr[RW];
#pragma unroll
        for (int i = 0; i < RW; i++) {
            const int last = (int)pos0 + r_t[i];   // last visible key of this row
            float a = s0[i] * p.scale, b = s1[i] * p.scale;
            if (p.softcap > 0.0f) { a = att_softcap(a, p.softcap, inv_cap2); b = att_softcap(b, p.softcap, inv_cap2); }
            const int da = last - (j0 + lane), db = da - 32;   // distances of the two keys
            if (p.r1) {
                a -= pen1[i] * __logf(1.0f + pen2[i] * (float)max(da, 0));
                b -= pen1[i] * __logf(1.0f + pen2[i] * (float)max(db, 0));
            }
            const bool va = r_ok[i] && da >= 0 && (p.window <= 0 || da < p.window || j0 + lane < p.keep_first);
            const bool vb = r_ok[i] && db >= 0 && (p.window <= 0 || db < p.window || j0 + lane + 32 < p.keep_first);
            a = va ? a : -1e30f; b = vb ? b : -1e30f;
            const float mt = warp_max(fmaxf(a, b));
            const float mn = fmaxf(m[i], mt);
            const float pa = va ? att_exp(a - mn) : 0.0f, pb = vb ? att_exp(b - mn) : 0.0f;
            corr[i] = att_exp(m[i] - mn);
            l[i] = l[i] * corr[i] + warp_sum(pa + pb);
            m[i] = mn;
            Ps[(size_t)(warp * RW + i) * ATT_KT + lane] = pa;
            Ps[(size_t)(warp * RW + i) * ATT_KT + lane + 32] = pb;
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < RW; i++)
#pragma unroll
            for (int c = 0; c < NI; c++) acc[i][c] *= corr[i];
        for (int j = 0; j < ATT_KT; j += 4) {
            float vv[4][NI];
#pragma unroll
            for (int jj = 0; jj < 4; jj++)
#pragma unroll
                for (int c = 0; c < NI; c++) vv[jj][c] = Vs[(size_t)(j + jj) * DVP + c * 32 + lane];
#pragma unroll
            for (int i = 0; i < RW; i++) {
                const float4 pv = *reinterpret_cast<const float4*>(Ps + (size_t)(warp * RW + i) * ATT_KT + j);
#pragma unroll
                for (int c = 0; c < NI; c++) {
                    acc[i][c] = fmaf(pv.x, vv[0][c], acc[i][c]); acc[i][c] = fmaf(pv.y, vv[1][c], acc[i][c]);
                    acc[i][c] = fmaf(pv.z, vv[2][c], acc[i][c]); acc[i][c] = fmaf(pv.w, vv[3][c], acc[i][c]);
                }
            }
        }
        __syncwarp();
    }
#pragma unroll
    for (int i = 0; i < RW; i++) {
        if (!r_ok[i]) continue;
        if (p.nsplit > 1) {
            float* dst = p.part + (((size_t)r_t[i] * p.H + r_h[i]) * p.nsplit + split) * (p.dv + 2);
            if (lane == 0) { dst[0] = m[i]; dst[1] = l[i]; }
#pragma unroll
            for (int c = 0; c < NI; c++)
                if (c * 32 + lane < p.dv) dst[2 + c * 32 + lane] = acc[i][c];
        } else {
            const float gt = p.gate ? p.gate[(size_t)r_t[i] * p.H + r_h[i]] : 1.0f;
            const float inv = gt * p.out_scale / l[i];
            AT* dst = p.out + (size_t)r_t[i] * p.out_ld + (size_t)r_h[i] * p.dv;
            const float* gl = p.gate_logits ? p.gate_logits + (size_t)r_t[i] * p.gate_ld + (size_t)r_h[i] * p.dv : nullptr;
#pragma unroll
            for (int c = 0; c < NI; c++)
                if (c * 32 + lane < p.dv) from_f(dst[c * 32 + lane], gl ? acc[i][c] * inv / (1.0f + expf(-gl[c * 32 + lane])) : acc[i][c] * inv);
        }
    }
}
// merges the key splits of a row: one warp per (token, head)
template <typename AT> struct AttnCombineParams {
    const float* part; const float* gate; AT* out;
    const float* gate_logits; int gate_ld;   // per-element sigmoid gates, as in AttnRowsParams
    int rows, H, dv, nsplit;   // rows = T * H
    int out_ld; float out_scale;             // as in AttnRowsParams
};
template <typename AT> __global__ void __launch_bounds__(128) attn_combine_kernel(const AttnCombineParams<AT> p) {
    pdl_launch();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= p.rows) return;
    const float* src = p.part + (size_t)r * p.nsplit * (p.dv + 2);
    // lane s holds split s (nsplit <= 32): its weight exp(m_s - max) is computed once and handed round by shuffles
    const float ms = lane < p.nsplit ? src[(size_t)lane * (p.dv + 2)] : -1e30f;
    const float mx = warp_max(ms);
    const float ws = lane < p.nsplit ? expf(ms - mx) : 0.0f;
    const float l = warp_sum(lane < p.nsplit ? src[(size_t)lane * (p.dv + 2) + 1] * ws : 0.0f);
    const float gt = p.gate ? p.gate[r] : 1.0f;
    const float inv = gt * p.out_scale / l;
    const float* gl = p.gate_logits ? p.gate_logits + (size_t)(r / p.H) * p.gate_ld + (size_t)(r % p.H) * p.dv : nullptr;
    AT* dst = p.out + (size_t)(r / p.H) * p.out_ld + (size_t)(r % p.H) * p.dv;
    for (int c0 = 0; c0 < p.dv; c0 += 32) {
        const int c = c0 + lane;
        float a = 0.0f;
#pragma unroll 8
        for (int s = 0; s < p.nsplit; s++) {
            const float w = __shfl_sync(0xffffffffu, ws, s);
            if (c < p.dv) a = fmaf(src[(size_t)s * (p.dv + 2) + 2 + c], w, a);
        }
        if (c < p.dv) from_f(dst[c], gl ? a * inv / (1.0f + expf(-gl[c])) : a * inv);
    }
}

// n columns of a wider f32 row, rounded to the operand type: out[t][0 .. n) = in[t * ld .. + n) (a slice of a fused projection
// that feeds the next matrix product)
template <typename AT> struct CastColsParams {
    const float* in; int ld;
    AT* out; int ldo;
    int n, total;   // total = T * n
};
template <typename AT> __global__ void __launch_bounds__(256) cast_cols_kernel(const CastColsParams<AT> p) {
    pdl_launch();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.total) return;
    const int t = i / p.n, c = i - t * p.n;
    from_f(p.out[(size_t)t * p.ldo + c], p.in[(size_t)t * p.ld + c]);
}

// f32 <- bf16 widening of a weight tensor (the f32 operand mode keeps its weights as f32 in HBM)
static __global__ void widen_bf16_kernel(float* dst, const __nv_bfloat16* src, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) dst[i] = __bfloat162float(src[i]);
}

}  // namespace dense
}  // namespace lmrs
