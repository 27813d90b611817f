// dense_gemm.cuh -- many-row bf16 matrix products of the unquantized models on the 5th-generation tensor cores:
//     out[T][O] (f32 accumulators) = A[T][K] (bf16) . W[O][K]^T (bf16),  then one of the epilogues of dense_ops.cuh
// tcgen05.mma kind::f16 (bf16 x bf16 -> f32) with the accumulator in TMEM, operands staged by TMA:
//   CTA tile 128 rows x 128 (or 64) accumulator columns, K walked 64 elements (128 bytes, one 128B-swizzle row) per stage
//   warp 0   TMA producer  A box [128 rows][128 B], B box [128 rows of W][128 B]  (GLU: 64 rows of gate + 64 rows of up)
//   warp 1   MMA issuer    4 x tcgen05.mma.cta_group::1.kind::f16 (M128 N128 K16) per stage, tcgen05.commit frees the stage
//   warps 2-5 epilogue     tcgen05.ld 32x32b.x32 (thread = one row x 32 columns), transposed through shared memory so that
//                          a warp writes 128 contiguous bytes per row: store*scale | x += ls*acc | glu(gate, up) | f(acc)
// The whole K range accumulates in TMEM (f32), so the accumulator is read once.  Ragged edges cost nothing extra: the
// tensor maps carry the true extents, TMA fills rows >= T, weight rows >= O and the K tail with zeros, and the epilogue
// masks its stores.  What the shape must satisfy: K and lda multiples of 8 elements (16-byte row pitch) and 16-byte
// aligned bases.  Three stages of 32 KB leave room for two CTAs per SM: one tile's epilogue runs under the other's MMAs.
// Every wait is bounded: a wait that runs out raises a flag in mapped host memory, the roles stop, in-flight copies are
// waited for (bounded again), TMEM is freed and the kernel returns; the next launch reports the flag.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <map>
#include <string>
#include <type_traits>

#include "common.cuh"
#include "dense_ops.cuh"

namespace lmrs {
namespace dense {

constexpr int TG_M = 128, TG_N = 128, TG_KB = 128 /* bytes of K per stage */, TG_STAGES = 3;
constexpr int TG_A_BYTES = TG_M * TG_KB, TG_B_BYTES = TG_N * TG_KB, TG_STAGE_BYTES = TG_A_BYTES + TG_B_BYTES;
constexpr int TG_THREADS = 64 + 128;
constexpr size_t TG_SMEM = 1024 + (size_t)TG_STAGES * TG_STAGE_BYTES + 256;
constexpr uint32_t TG_SPIN_LIMIT = 1u << 24;   // try_wait calls (each suspends for a while) before a wait gives up

struct TcGemmParams {
    int T, K, O;
    EpiParams<__nv_bfloat16> e;
    int* err;   // mapped host word: set to 1 when a wait ran out
    // grouped form (one matrix per expert over rows sorted by expert): blockIdx.z = group z owns rows grp[z] .. grp[z+1] of A and
    // of the output and rows z*O .. z*O+O of the weight tensor map; null: one matrix for all T rows
    const int* grp;
};

DN_DEVINL bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < TG_SPIN_LIMIT; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
DN_DEVINL void tg_tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_u32(dst)),
                 "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}
// K-major operand tile with rows of exactly 128 bytes under SWIZZLE_128B: 8-row atoms 1024 bytes apart
DN_DEVINL uint64_t tg_desc_sw128(const void* smem_tile) {
    const uint32_t addr = smem_u32(smem_tile);
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// instruction descriptor: D = f32, A = B = bf16, both K-major, M = 128, N = BN, dense
template <int BN> __host__ __device__ constexpr uint32_t tg_idesc() {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TG_M >> 4) << 24);
}
DN_DEVINL void tg_mma(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
DN_DEVINL void tg_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
DN_DEVINL void tg_tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}

// EPI_GLU: the B tile is 64 rows of the gate matrix followed by the same 64 rows of the up matrix, so accumulator
// columns c and c + 64 belong to output column n0 + c and the CTA produces 64 output columns; otherwise 128.
// BN = accumulator columns per CTA: 128, or 64 for matrices with so few output rows that 128-wide tiles would leave
// most SMs without a CTA (output and down projections at short prompts).
template <int EPI, int BN>
__global__ void __launch_bounds__(TG_THREADS, 2)
gemm_bf16_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const __grid_constant__ CUtensorMap tm_b2,
                    const TcGemmParams p) {
    constexpr bool GLU = EPI == EPI_GLU;
    static_assert(BN == 128 || (BN == 64 && !GLU), "tile width");
    constexpr int OUT_COLS = GLU ? 64 : BN;
    constexpr uint32_t STAGE_TX = TG_A_BYTES + BN * TG_KB;   // bytes one stage receives (the ring keeps 32 KB slots)
    extern __shared__ uint8_t tg_raw[];
    uint8_t* sm = tg_raw + (((smem_u32(tg_raw) + 1023u) & ~1023u) - smem_u32(tg_raw));
    uint8_t* tiles = sm;
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + (size_t)TG_STAGES * TG_STAGE_BYTES);
    uint64_t* empty = full + TG_STAGES;
    uint64_t* tfull = empty + TG_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tfull + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int m0 = blockIdx.y * TG_M, row_end = p.T, wrow0 = 0;
    const int n0 = blockIdx.x * OUT_COLS;
    if (p.grp) {   // tiles past the group's last row leave before anything is set up (the whole CTA takes this branch)
        m0 += p.grp[blockIdx.z];
        row_end = p.grp[blockIdx.z + 1];
        wrow0 = (int)blockIdx.z * p.O;
        if (m0 >= row_end) return;
    }
    const int KS = (p.K * 2 + TG_KB - 1) / TG_KB;   // stages over K

    if (threadIdx.x == 0) {
        for (int s = 0; s < TG_STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(tfull, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {   // ---- TMA producer ----
            int issued = 0;
            for (int g = 0; g < KS; g++) {
                const int s = g % TG_STAGES;
                if (!mbar_wait_bounded(&empty[s], ((g / TG_STAGES) & 1) ^ 1, abort_flag)) break;
                uint8_t* a_t = tiles + (size_t)s * TG_STAGE_BYTES;
                mbar_expect_tx(&full[s], STAGE_TX);
                tg_tma_load_2d(a_t, &tm_a, g * TG_KB, m0, &full[s]);
                if (GLU) {
                    tg_tma_load_2d(a_t + TG_A_BYTES, &tm_b, g * TG_KB, wrow0 + n0, &full[s]);
                    tg_tma_load_2d(a_t + TG_A_BYTES + 64 * TG_KB, &tm_b2, g * TG_KB, wrow0 + n0, &full[s]);
                } else {
                    tg_tma_load_2d(a_t + TG_A_BYTES, &tm_b, g * TG_KB, wrow0 + n0, &full[s]);
                }
                issued = g + 1;
            }
            if (*abort_flag) {   // gave up somewhere: let the copies already requested land before shared memory goes away
                for (int g = issued > TG_STAGES ? issued - TG_STAGES : 0; g < issued; g++)
                    for (uint32_t i = 0; i < TG_SPIN_LIMIT && !mbar_try_wait(&full[g % TG_STAGES], (g / TG_STAGES) & 1); i++) {}
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {   // ---- MMA issuer ----
            const uint32_t idesc = tg_idesc<BN>();
            bool ok = true;
            for (int g = 0; g < KS && ok; g++) {
                const int s = g % TG_STAGES;
                ok = mbar_wait_bounded(&full[s], (g / TG_STAGES) & 1, abort_flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint8_t* a_t = tiles + (size_t)s * TG_STAGE_BYTES;
                const uint64_t da = tg_desc_sw128(a_t), db = tg_desc_sw128(a_t + TG_A_BYTES);
#pragma unroll
                for (int k = 0; k < TG_KB / 32; k++)   // 16 bf16 = 32 bytes along K inside the swizzle atom
                    tg_mma(tmem_base, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (g > 0 || k > 0) ? 1u : 0u);
                tg_commit(&empty[s]);
            }
            if (ok) tg_commit(tfull);
        }
    } else {   // ---- epilogue: TMEM lane quadrant = warp % 4 ----
        // tcgen05.ld hands a thread one ROW of the tile (32 consecutive columns per load).  Writing rows from there would
        // touch 32 different cache lines per instruction, so each 32 x 32 block goes through shared memory (the operand
        // ring is idle by now: every MMA that read it has completed) and leaves with lane = column: 128 contiguous bytes
        // per row, loads of the residual batched eight rows ahead of their stores.
        const int quad = warp & 3;
        float* stg = reinterpret_cast<float*>(tiles) + (size_t)(warp - 2) * 32 * 33;
        const bool ok = mbar_wait_bounded(tfull, 0, abort_flag);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
#pragma unroll 1
            for (int c0 = 0; c0 < OUT_COLS; c0 += 32) {
                uint32_t v[32], u[GLU ? 32 : 1];
                tg_tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, v);
                if constexpr (GLU) tg_tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(64 + c0), u);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    float val = __uint_as_float(v[j]);
                    if constexpr (GLU) val = glu_apply(p.e, val, __uint_as_float(u[j]));
                    if constexpr (EPI == EPI_ACT) val = act_apply(p.e, val);
                    stg[lane * 33 + j] = val;
                }
                __syncwarp();
                const int o = n0 + c0 + lane;
                const int t0 = m0 + quad * 32;
                if (o < p.O) {
                    if constexpr (EPI == EPI_STORE) {
                        float* __restrict__ dst = p.e.out + (size_t)t0 * p.e.ldo + o;
                        const float bias = p.e.bias ? p.e.bias[o] : 0.0f;
#pragma unroll 8
                        for (int r = 0; r < 32; r++)
                            if (t0 + r < row_end) dst[(size_t)r * p.e.ldo] = p.e.bias ? stg[r * 33 + lane] * p.e.scale + bias : stg[r * 33 + lane] * p.e.scale;
                    } else if constexpr (EPI == EPI_RESID) {
                        float* __restrict__ dst = p.e.out + (size_t)t0 * p.e.ldo + o;
                        const float lsv = p.e.ls[o], lbv = p.e.lb ? p.e.lb[o] : 0.0f;
                        const float alpha = p.e.tanh_alpha ? *p.e.tanh_alpha : 0.0f;
#pragma unroll 1
                        for (int r0 = 0; r0 < 32; r0 += 8) {
                            float x[8];
#pragma unroll
                            for (int r = 0; r < 8; r++) x[r] = (t0 + r0 + r < row_end) ? dst[(size_t)(r0 + r) * p.e.ldo] : 0.0f;
#pragma unroll
                            for (int r = 0; r < 8; r++)
                                if (t0 + r0 + r < row_end) {
                                    float a = stg[(r0 + r) * 33 + lane];
                                    if (p.e.tanh_alpha) a = tanhf(alpha * a);
                                    dst[(size_t)(r0 + r) * p.e.ldo] = p.e.lb ? x[r] + (lsv * a + lbv) : x[r] + lsv * a;
                                }
                        }
                    } else {
                        __nv_bfloat16* __restrict__ dst = p.e.act + (size_t)t0 * p.e.lda + o;
#pragma unroll 8
                        for (int r = 0; r < 32; r++)
                            if (t0 + r < row_end) dst[(size_t)r * p.e.lda] = __float2bfloat16_rn(stg[r * 33 + lane]);
                    }
                }
                __syncwarp();
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(BN) : "memory");
    }
    if (threadIdx.x == 0 && *abort_flag && p.err) *p.err = 1;
}

// ---- host side ------------------------------------------------------------------------------------------------------------
typedef CUresult (*TgEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
struct DenseGemmCtx {
    int sms = 148;
    TgEncodeTiledFn enc = nullptr;
    bool tried = false;
    int* h_err = nullptr;   // mapped, pinned
    int* d_err = nullptr;
    std::map<std::pair<const void*, int>, CUtensorMap> wmaps;   // (weight matrix, box rows) -> tensor map
    bool attr_set[4][2] = {};
    ~DenseGemmCtx() { if (h_err) cudaFreeHost(h_err); }
};
// a [rows][row_bytes used of pitch_bytes] byte matrix, box 128 bytes x box_rows rows, 128B swizzle, zeros outside
inline bool tg_make_map(DenseGemmCtx& c, CUtensorMap* map, const void* base, size_t row_bytes, size_t pitch_bytes, size_t rows, int box_rows) {
    cuuint64_t gdim[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
    cuuint64_t gstride[1] = {(cuuint64_t)pitch_bytes};
    cuuint32_t box[2] = {(cuuint32_t)TG_KB, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return c.enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
template <typename AT, typename WT> inline bool dense_gemm_usable(int T, int K, int O, int lda) {
    if (!std::is_same<AT, __nv_bfloat16>::value || !std::is_same<WT, __nv_bfloat16>::value) return false;
    return T >= 2 && K % 8 == 0 && lda % 8 == 0 && O >= 1;
}
// returns 0 on success, 1 on failure (message in err), -1 when the kernel cannot be used here (caller falls back)
// n_groups > 0: the grouped form -- `w` (and `w2`) hold n_groups matrices [O][K] back to back, `grp` (device) the row offsets of the
// groups in A and in the output, T the total number of rows and max_group_rows a bound on the rows of one group
template <typename AT, typename WT, int EPI>
inline int dense_gemm_launch(DenseGemmCtx& c, cudaStream_t st, int T, const AT* a, int lda, const WT* w, const WT* w2, int K, int O,
                             const EpiParams<AT>& e, std::string& err, const int* grp = nullptr, int n_groups = 0, int max_group_rows = 0) {
    if constexpr (!std::is_same<AT, __nv_bfloat16>::value || !std::is_same<WT, __nv_bfloat16>::value) {
        return -1;
    } else {
        if (!c.tried) {
            c.tried = true;
            void* fp = nullptr;
            cudaDriverEntryPointQueryResult q;
            if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fp, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
                c.enc = (TgEncodeTiledFn)fp;
            if (c.enc && cudaHostAlloc(&c.h_err, sizeof(int), cudaHostAllocMapped) == cudaSuccess) {
                *c.h_err = 0;
                if (cudaHostGetDevicePointer(&c.d_err, c.h_err, 0) != cudaSuccess) c.enc = nullptr;
            } else {
                c.enc = nullptr;
            }
        }
        if (!c.enc) return -1;
        if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) || (w2 && (reinterpret_cast<uintptr_t>(w2) & 15))) return -1;
        if (*c.h_err) { err = "a tensor-core matrix product gave up waiting on one of its barriers (device status flag set)"; return 1; }
        constexpr bool GLU = EPI == EPI_GLU;
        // 64-wide tiles when 128-wide ones would not give every SM a CTA
        const size_t w_rows = n_groups > 0 ? (size_t)n_groups * O : (size_t)O;
        const bool narrow = !GLU && O > 64 && ((O + 127) / 128) * ((T + TG_M - 1) / TG_M) < c.sms;
        const int box_rows = (GLU || narrow) ? 64 : 128;
        auto wmap = [&](const void* base, CUtensorMap* out) {
            auto key = std::make_pair(base, box_rows * 1000003 + (int)(w_rows % 1000003));
            auto it = c.wmaps.find(key);
            if (it == c.wmaps.end()) {
                CUtensorMap m;
                if (!tg_make_map(c, &m, base, (size_t)K * 2, (size_t)K * 2, w_rows, box_rows)) return false;
                it = c.wmaps.emplace(key, m).first;
            }
            *out = it->second;
            return true;
        };
        CUtensorMap ta, tb, tb2;
        if (!tg_make_map(c, &ta, a, (size_t)K * 2, (size_t)lda * 2, (size_t)T, 128)) return -1;
        if (!wmap(w, &tb)) return -1;
        tb2 = tb;
        if (GLU && !wmap(w2, &tb2)) return -1;
        if (!c.attr_set[EPI][narrow]) {
            cudaError_t ae = narrow ? cudaFuncSetAttribute(gemm_bf16_tc_kernel<EPI, GLU ? 128 : 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TG_SMEM)
                                    : cudaFuncSetAttribute(gemm_bf16_tc_kernel<EPI, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TG_SMEM);
            if (ae != cudaSuccess) { err = "cudaFuncSetAttribute(gemm_bf16_tc_kernel) failed"; return 1; }
            c.attr_set[EPI][narrow] = true;
        }
        TcGemmParams p{};
        p.T = T; p.K = K; p.O = O; p.e = e; p.err = c.d_err; p.grp = n_groups > 0 ? grp : nullptr;
        const int out_cols = (GLU || narrow) ? 64 : TG_N;
        const int rows_y = n_groups > 0 ? std::min(T, max_group_rows) : T;
        const dim3 grid((O + out_cols - 1) / out_cols, (rows_y + TG_M - 1) / TG_M, n_groups > 0 ? n_groups : 1);
        if (narrow) gemm_bf16_tc_kernel<EPI, GLU ? 128 : 64><<<grid, TG_THREADS, TG_SMEM, st>>>(ta, tb, tb2, p);
        else gemm_bf16_tc_kernel<EPI, 128><<<grid, TG_THREADS, TG_SMEM, st>>>(ta, tb, tb2, p);
        cudaError_t ce = cudaGetLastError();
        if (ce != cudaSuccess) { err = std::string("gemm_bf16_tc_kernel: ") + cudaGetErrorString(ce); return 1; }
        return 0;
    }
}

}  // namespace dense
}  // namespace lmrs
