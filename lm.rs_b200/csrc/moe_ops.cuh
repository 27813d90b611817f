// moe_ops.cuh -- a feed-forward made of routed experts, around the matrix kernels of dense_ops.cuh / dense_gemm.cuh:
//   moe_logits_kernel    router logits in f32 (f32 router matrix)
//   moe_topk_kernel      score = sigmoid(logit), or the softmax over all logits; the `top` experts with the largest
//                        score + correction[e] are chosen, their weights are score / (sum of chosen scores + 1e-20) * scale
//   moe_sort_kernel      (token, choice) pairs counted and sorted by expert: row offsets per expert, the slot of every pair,
//                        the token of every slot
//   moe_gather_kernel    the normalised rows copied into expert order (the grouped matrix kernels then see one contiguous row
//                        range per expert)
//   moe_combine_kernel   x += f(sum over the token's choices of weight * expert output), f = a tanh norm on the way into the
//                        residual (or the identity); or the sum stored for a norm that needs statistics.  Experts beyond
//                        the ones with matrices are identity experts (their output is the token's input row); a shared
//                        expert's output row can be added
//   moe_combine_layernorm_kernel   the same sum through a layer norm into the residual stream: one CTA per token, or a
//                        single token's columns over several CTAs of which the last one to finish applies the norm
// A one-row step needs no sorting: the one-row matrix kernel takes the chosen experts from the router's device-side list.
#pragma once
#include "dense_ops.cuh"

namespace lmrs {
namespace dense {

template <typename AT> struct MoeRouterParams {
    const AT* h; int ld;          // [T][width] normalised input (operand type), or null:
    const float* x; TanhNorm tn;  // ... the residual row, normalised here (tanh norm) and rounded to the operand type
    const float* router;          // [E][width]
    const float* correction;      // [E], added for the choice only
    int E, top, width;
    int softmax;                  // 0: score = sigmoid(logit); 1: scores = softmax over the E logits; 2: the largest logits are
                                  // chosen and the weights are the softmax over the chosen logits only (times scale)
    const float* bias;            // [E] or null: added to the router logits
    float scale;
    float* z;                     // [T][E] router logits (scratch between the two kernels)
    int* idx; float* wts;         // [T][top]
};
// logits: one warp per (token, expert), so that a single token still spreads over E warps on many SMs
template <typename AT> __global__ void __launch_bounds__(128) moe_logits_kernel(const MoeRouterParams<AT> p) {
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x, lane = threadIdx.x & 31;
    const int e = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (e >= p.E) return;
    const float* w = p.router + (size_t)e * p.width;
    float a = 0.0f;
    if (p.h) {
        const AT* h = p.h + (size_t)t * p.ld;
#pragma unroll 8
        for (int c = lane; c < p.width; c += 32) a = fmaf(w[c], to_f(h[c]), a);
    } else {
        const float* x = p.x + (size_t)t * p.ld;
        const float alpha = *p.tn.alpha;
#pragma unroll 8
        for (int c = lane; c < p.width; c += 32) { AT r; from_f(r, tanhnorm_apply(p.tn, alpha, c, x[c])); a = fmaf(w[c], to_f(r), a); }
    }
    a = warp_sum(a);
    if (lane == 0) p.z[(size_t)t * p.E + e] = p.bias ? a + p.bias[e] : a;
}
// choice: one warp per token
template <typename AT> __global__ void __launch_bounds__(32) moe_topk_kernel(const MoeRouterParams<AT> p) {
    extern __shared__ __align__(16) float mr_sm[];
    float* score = mr_sm;            // [E] sigmoid(logit)
    float* choice = score + p.E;     // [E] score + correction; -inf once chosen
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x, lane = threadIdx.x;
    float zmax = -INFINITY, zsum = 0.0f;
    if (p.softmax == 1) {
        for (int e = lane; e < p.E; e += 32) zmax = fmaxf(zmax, p.z[(size_t)t * p.E + e]);
        zmax = warp_max(zmax);
        for (int e = lane; e < p.E; e += 32) zsum += expf(p.z[(size_t)t * p.E + e] - zmax);
        zsum = warp_sum(zsum);
    }
    for (int e = lane; e < p.E; e += 32) {
        const float z = p.z[(size_t)t * p.E + e];
        const float sg = p.softmax == 2 ? z : (p.softmax == 1 ? expf(z - zmax) / zsum : 1.0f / (1.0f + expf(-z)));
        score[e] = sg;
        choice[e] = sg + (p.correction ? p.correction[e] : 0.0f);
    }
    __syncwarp();
    float sum = 0.0f;
    for (int k = 0; k < p.top; k++) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < p.E; e += 32)
            if (choice[e] > best) { best = choice[e]; bi = e; }   // ascending e: the lowest index wins a tie inside a lane
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        const float sg = score[bi];
        sum += sg;
        if (lane == 0) { p.idx[(size_t)t * p.top + k] = bi; p.wts[(size_t)t * p.top + k] = sg; choice[bi] = -INFINITY; }
        __syncwarp();
    }
    if (p.softmax == 2) {   // the first choice holds the largest logit: weights exp(z_k - z_0) / sum
        __syncwarp();
        const float z0 = p.wts[(size_t)t * p.top];
        float es = 0.0f;
        for (int k = lane; k < p.top; k += 32) es += expf(p.wts[(size_t)t * p.top + k] - z0);
        es = warp_sum(es);
        for (int k = lane; k < p.top; k += 32) p.wts[(size_t)t * p.top + k] = expf(p.wts[(size_t)t * p.top + k] - z0) / es * p.scale;
        return;
    }
    const float f = p.scale / (sum + 1e-20f);
    for (int k = lane; k < p.top; k += 32) p.wts[(size_t)t * p.top + k] *= f;
}

// n = T * top pairs.  One CTA: histogram, exclusive scan, placement.  Which pair of an expert gets which of the expert's
// slots depends on the order the atomics land in; every row is computed on its own, so the results do not.
struct MoeSortParams {
    const int* idx; int n, E, top;
    int* grp;       // [E + 1]
    int* slot;      // [n]: slot of pair (t, k)
    int* row_of;    // [n]: token of a slot
};
static __global__ void __launch_bounds__(1024) moe_sort_kernel(const MoeSortParams p) {
    extern __shared__ int ms_sm[];   // [E] counts, then [E] cursors
    int* cnt = ms_sm;
    int* cur = cnt + p.E;
    pdl_launch();
    pdl_wait();
    for (int e = threadIdx.x; e < p.E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < p.n; i += blockDim.x) atomicAdd(&cnt[p.idx[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int a = 0;
        for (int e = 0; e < p.E; e++) { p.grp[e] = a; cur[e] = a; a += cnt[e]; }
        p.grp[p.E] = a;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < p.n; i += blockDim.x) {
        const int s = atomicAdd(&cur[p.idx[i]], 1);
        p.slot[i] = s;
        p.row_of[s] = i / p.top;
    }
}

template <typename AT> struct MoeGatherParams {
    const AT* h; int ld; const int* row_of; AT* out; int width;
};
template <typename AT> __global__ void __launch_bounds__(128) moe_gather_kernel(const MoeGatherParams<AT> p) {
    pdl_launch();
    pdl_wait();
    const AT* src = p.h + (size_t)p.row_of[blockIdx.x] * p.ld;
    AT* dst = p.out + (size_t)blockIdx.x * p.width;
    for (int c = threadIdx.x; c < p.width; c += blockDim.x) dst[c] = src[c];
}

struct MoeCombineParams {
    const float* y;           // [slots][width] expert outputs
    const int* slot;          // [T][top] slot of every pair, or null: pair (t, k) sits in slot t*top + k
    const float* wts;         // [T][top]
    float* x; int ldx;        // residual stream
    TanhNorm n;               // n.alpha null: x += sum;  else x += tanh(alpha * sum) * w + b
    int top, width;
    const int* idx; int n_real;        // idx set: a pair whose expert idx[t][k] >= n_real is an identity expert ...
    const float* xin; int ld_in;       // ... whose output is row t of xin
    const float* add;                  // or null: [T][width] added to the sum (a shared expert's output)
    float* out; int ldo;               // when set: the sum is stored here and x is left alone
};
// the weighted sum of one token's expert outputs at column c
DN_DEVINL float moe_combined(const MoeCombineParams& p, int t, int c) {
    float a = p.add ? p.add[(size_t)t * p.width + c] : 0.0f;
    for (int k = 0; k < p.top; k++) {
        const float w = p.wts[(size_t)t * p.top + k];
        if (p.idx && p.idx[(size_t)t * p.top + k] >= p.n_real) { a = fmaf(w, p.xin[(size_t)t * p.ld_in + c], a); continue; }
        const int s = p.slot ? p.slot[(size_t)t * p.top + k] : t * p.top + k;
        a = fmaf(w, p.y[(size_t)s * p.width + c], a);
    }
    return a;
}
static __global__ void __launch_bounds__(256) moe_combine_kernel(const MoeCombineParams p) {
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    const float alpha = p.n.alpha ? *p.n.alpha : 0.0f;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < p.width; c += gridDim.y * blockDim.x) {
        const float a = moe_combined(p, t, c);
        if (p.out) p.out[(size_t)t * p.ldo + c] = a;
        else p.x[(size_t)t * p.ldx + c] += p.n.alpha ? tanhnorm_apply(p.n, alpha, c, a) : a;
    }
}
// the same sum sent through a layer norm into the residual stream, x <- x + ls * LN(sum) w, and x again in the operand type
// to h.  The norm needs the whole row: with gridDim.y == 1 one CTA per token computes the row and holds it in registers.  A
// single token (gridDim.x == 1) may instead spread its columns over gridDim.y CTAs, which store the sums in c.out; each takes a
// ticket from *counter when its stores are done and the one that comes last applies the norm (nobody waits; that CTA puts
// the counter back to zero).
template <typename AT> struct MoeCombineNormParams {
    MoeCombineParams c;
    const float* w; const float* ls; float eps;
    AT* h; int ldh;
    unsigned int* counter;
};
template <typename AT> __global__ void __launch_bounds__(256) moe_combine_layernorm_kernel(const MoeCombineNormParams<AT> p) {
    __shared__ float red[33];
    __shared__ unsigned int last;
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    float* xr = p.c.x + (size_t)t * p.c.ldx;
    if (gridDim.y == 1) {
        layernorm_row<AT>([&](int c) { return moe_combined(p.c, t, c); }, p.c.width, p.w, p.eps, red, xr, p.ls, nullptr, p.h + (size_t)t * p.ldh);
        return;
    }
    float* row = p.c.out + (size_t)t * p.c.ldo;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < p.c.width; c += gridDim.y * blockDim.x) row[c] = moe_combined(p.c, t, c);
    __threadfence();   // this thread's stores of the row before the ticket
    __syncthreads();
    if (threadIdx.x == 0) last = atomicAdd(p.counter, 1u) == gridDim.y - 1 ? 1u : 0u;
    __syncthreads();
    if (!last) return;
    __threadfence();
    layernorm_row<AT>([&](int c) { return __ldcg(row + c); }, p.c.width, p.w, p.eps, red, xr, p.ls, nullptr, p.h + (size_t)t * p.ldh);
    if (threadIdx.x == 0) *p.counter = 0u;
}

}  // namespace dense
}  // namespace lmrs
