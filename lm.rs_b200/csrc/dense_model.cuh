// dense_model.cuh -- what every folder architecture (arch.h) with unquantized weights shares: device allocations, tensor
// lookup and upload in the operand type, kernel launch helpers (matrix products that pick the tensor-core, CUDA-core or
// one-row kernel; attention; batched and grouped products), the many-token step that walks a prompt portion in chunks and
// gathers the wanted rows for the head, and the decode step replayed from a CUDA graph per position bucket.  An
// architecture derives from DenseModel, loads its tensors, and implements run_layers() / head_rows() by composing the
// kernels of dense_ops.cuh, mixer_ops.cuh and moe_ops.cuh.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <set>
#include <string>
#include <vector>

#include "arch.h"
#include "dense_gemm.cuh"
#include "dense_ops.cuh"
#include "safetensors.h"

namespace lmrs {

using namespace dense;

static inline float bf16_bits_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

#define GCK(call)                                                                                                      \
    do {                                                                                                               \
        cudaError_t e_ = (call);                                                                                       \
        if (e_ != cudaSuccess) {                                                                                       \
            error = std::string(#call) + ": " + cudaGetErrorString(e_) + " (" + __FILE__ + ":" + std::to_string(__LINE__) + ")"; \
            return 1;                                                                                                  \
        }                                                                                                              \
    } while (0)

template <typename AT, typename WT> class DenseModel : public ArchModel {
  public:
    using ArchModel::error;
    using ArchModel::launches;
    using ArchModel::info;
    using ArchModel::d_logits;
    std::vector<void*> owned;   // every device allocation
    int width = 0, vocab = 0;
    uint32_t max_tokens = 0;
    int sms = 148;
    uint32_t* d_tokens = nullptr;   // [max_tokens] token history
    size_t cap = 0;                 // rows the scratch buffers hold
    float* x = nullptr;             // [cap][width] residual stream
    AT* hn = nullptr;               // [cap][width] normalised rows for the head
    uint32_t* d_rows = nullptr;
    float* d_head_tmp = nullptr;
    size_t head_tmp_rows = 0;
    static constexpr int MAX_SPLIT = 32;
    bool keep_layers = false;
    float* d_layer_out = nullptr;
    size_t layer_out_rows = 0, layer_out_cap = 0;
    size_t chunk_rows = 2048;
    int use_tc = 1;   // tcgen05 GEMM for aligned bf16 shapes (0: always the CUDA-core kernel)
    dense::DenseGemmCtx gemm_ctx;
    struct GraphEntry { cudaGraphExec_t exec = nullptr; uint64_t kernels = 0; };
    std::map<int, GraphEntry> graphs;   // decode step per position bucket
    std::set<int> warmed;
    const StepParams* graph_step = nullptr;
    // programmatic dependent launch of the decode chain is an option, off by default: measured slower here (1.32 vs 1.14 ms
    // per step at 16 layers of width 2048): the early-launched CTAs of the next kernels sit on the SMs while they wait
    int use_graph = 1, use_pdl = 0;

    // what an architecture implements
    virtual size_t n_layers() const = 0;
    virtual int ensure_scratch(size_t rows) = 0;   // (re)allocate x, hn, d_rows and its own buffers for `rows` rows; sets cap
    // the layers over T rows at positions pos ..; x holds the residual stream on return
    virtual int run_layers(cudaStream_t st, int T, const dense::PosSrc& ps, uint32_t pos_hint) = 0;
    // final norm + head over `m` rows of x given by rows_dev[0..m) (null with m == 1: row 0) -> out [m][vocab]
    virtual int head_rows(cudaStream_t st, int m, const uint32_t* rows_dev, float* out) = 0;
    virtual void set_model_option(const char*, int) {}
    // called before a step of n tokens at position pos is enqueued (models with state that is not addressed by position check it here)
    virtual int begin_step(uint32_t pos, size_t n) { (void)pos; (void)n; return 0; }

    ~DenseModel() override {
        drop_graphs();
        for (void* p : owned) cudaFree(p);
    }
    template <typename T> int dalloc(T** p, size_t n) {
        void* v = nullptr;
        GCK(cudaMalloc(&v, std::max<size_t>(n, 1) * sizeof(T)));
        owned.push_back(v);
        *p = static_cast<T*>(v);
        return 0;
    }
    void dfree(void* p) {
        if (!p) return;
        owned.erase(std::remove(owned.begin(), owned.end(), p), owned.end());
        cudaFree(p);
    }

    // ---- weights ------------------------------------------------------------------------------------------------------
    int need(const SafeTensors& st, const std::string& name, std::vector<int64_t> shape, const StTensor** out) {
        const StTensor* t = st.find(name);
        if (!t) { error = "tensor '" + name + "' is missing"; return 1; }
        if (t->dtype != "BF16" && t->dtype != "F32") { error = "tensor '" + name + "': dtype " + t->dtype + " is not BF16 or F32"; return 1; }
        if (t->shape != shape) {
            error = "tensor '" + name + "' has shape [";
            for (int64_t d : t->shape) error += std::to_string(d) + ",";
            error += "], the configuration wants [";
            for (int64_t d : shape) error += std::to_string(d) + ",";
            error += "]";
            return 1;
        }
        *out = t;
        return 0;
    }
    // a matrix (or a block of rows of a concatenated matrix) in the operand type
    int upload_w(const StTensor* t, WT* dst) {
        const size_t n = t->numel();
        if (n == 0) return 0;
        const bool src_bf16 = t->dtype == "BF16";
        if (std::is_same<WT, __nv_bfloat16>::value) {
            if (src_bf16) { GCK(cudaMemcpy(dst, t->data, n * 2, cudaMemcpyHostToDevice)); }
            else {
                std::vector<__nv_bfloat16> tmp(n);
                const float* s = reinterpret_cast<const float*>(t->data);
                for (size_t i = 0; i < n; i++) tmp[i] = __float2bfloat16_rn(s[i]);
                GCK(cudaMemcpy(dst, tmp.data(), n * 2, cudaMemcpyHostToDevice));
            }
        } else {
            if (src_bf16) {
                __nv_bfloat16* stage = nullptr;
                GCK(cudaMalloc(&stage, n * 2));
                cudaError_t e = cudaMemcpy(stage, t->data, n * 2, cudaMemcpyHostToDevice);
                if (e == cudaSuccess) {
                    widen_bf16_kernel<<<(unsigned)std::min<size_t>((n + 255) / 256, 4096), 256>>>(reinterpret_cast<float*>(dst), stage, n);
                    e = cudaDeviceSynchronize();
                }
                cudaFree(stage);
                GCK(e);
            } else {
                GCK(cudaMemcpy(dst, t->data, n * 4, cudaMemcpyHostToDevice));
            }
        }
        return 0;
    }
    int upload_f32(const StTensor* t, float** dst) {   // small vectors that are always used in f32
        const size_t n = t->numel();
        std::vector<float> tmp(std::max<size_t>(n, 1));
        if (t->dtype == "BF16") {
            const uint16_t* s = reinterpret_cast<const uint16_t*>(t->data);
            for (size_t i = 0; i < n; i++) tmp[i] = bf16_bits_to_f32(s[i]);
        } else {
            memcpy(tmp.data(), t->data, n * 4);
        }
        if (dalloc(dst, n)) return 1;
        GCK(cudaMemcpy(*dst, tmp.data(), n * 4, cudaMemcpyHostToDevice));
        return 0;
    }

    // ---- launches -------------------------------------------------------------------------------------------------------
    int check_launch(const char* what) {
        launches++;
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) { error = std::string(what) + ": " + cudaGetErrorString(e); return 1; }
        return 0;
    }
    // every kernel launch of the model; `pdl`: with the programmatic-dependent-launch attribute (decode chain)
    template <typename... KArgs, typename... Args>
    int launch_k(const char* what, cudaStream_t st, bool pdl, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args... args) {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pdl ? 1 : 0;
        launches++;
        cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, args...);
        if (e != cudaSuccess) { error = std::string(what) + ": " + cudaGetErrorString(e); return 1; }
        return 0;
    }
    bool pdl_now = false;   // set while a decode step is being enqueued
    template <typename K> int optin(K kernel, size_t smem) {
        if (smem <= 48 * 1024) return 0;
        static std::map<const void*, size_t> done;
        auto it = done.find((const void*)kernel);
        if (it != done.end() && it->second >= smem) return 0;
        GCK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        done[(const void*)kernel] = smem;
        return 0;
    }

    // cos/sin of position * f_i for every cached position, times `mult`, made on the host in f64: [max_tokens][f.size()]
    // each; one pair of tables per distinct key (layers with the same rotary configuration share them)
    std::map<std::string, std::pair<float*, float*>> angle_tabs;
    int angle_tables(const std::string& key, const std::vector<double>& f, double mult, const float** cos_out, const float** sin_out) {
        auto it = angle_tabs.find(key);
        if (it == angle_tabs.end()) {
            const size_t half = f.size();
            std::vector<float> c((size_t)max_tokens * std::max<size_t>(half, 1)), s(c.size());
            for (size_t i = 0; i < half; i++)
                for (uint32_t p = 0; p < max_tokens; p++) {
                    const double a = (double)p * f[i];
                    c[(size_t)p * half + i] = (float)(cos(a) * mult);
                    s[(size_t)p * half + i] = (float)(sin(a) * mult);
                }
            float *dc = nullptr, *ds = nullptr;
            if (dalloc(&dc, c.size()) || dalloc(&ds, s.size())) return 1;
            GCK(cudaMemcpy(dc, c.data(), c.size() * 4, cudaMemcpyHostToDevice));
            GCK(cudaMemcpy(ds, s.data(), s.size() * 4, cudaMemcpyHostToDevice));
            it = angle_tabs.emplace(key, std::make_pair(dc, ds)).first;
        }
        *cos_out = it->second.first;
        *sin_out = it->second.second;
        return 0;
    }

    // out = a . w^T with an epilogue; T rows.  One row: the streaming kernel; many rows: tensor cores when the shape
    // allows, else CUDA cores.
    template <int EPI> int matmul(cudaStream_t st, int T, const AT* a, int lda, const WT* w, const WT* w2, int K, int O, const EpiParams<AT>& e) {
        if (T == 1) {
            GemvRowsParams<AT, WT> p{};
            p.a = a; p.w = w; p.w2 = w2; p.K = K; p.O = O; p.e = e;
            return launch_gemv<EPI, NORM_NONE>(st, p);
        }
        if (use_tc && dense_gemm_usable<AT, WT>(T, K, O, lda)) {
            int rc = dense_gemm_launch<AT, WT, EPI>(gemm_ctx, st, T, a, lda, w, w2, K, O, e, error);
            if (rc >= 0) { launches++; return rc; }
        }
        GemmTiledParams<AT, WT> p{};
        p.a = a; p.lda = lda; p.w = w; p.w2 = w2; p.T = T; p.K = K; p.O = O; p.e = e;
        gemm_tiled_kernel<AT, WT, EPI><<<dim3((O + 63) / 64, (T + 63) / 64), 256, 0, st>>>(p);
        return check_launch("gemm_tiled_kernel");
    }
    // nb products at once, one matrix per batch entry z (a head): out[:, z*o_bs ..] = a[:, z*a_bs ..] . (w + z*w_bs)^T.  The
    // matrices are small (a head's share of a projection), so the CUDA-core kernels serve both operand types.
    template <int EPI> int matmul_batched(cudaStream_t st, int T, int nb, const AT* a, int lda, long long a_bs, const WT* w, long long w_bs,
                                          int K, int O, const EpiParams<AT>& e, long long o_bs) {
        if (T == 1) {
            GemvRowsParams<AT, WT> p{};
            p.a = a; p.w = w; p.K = K; p.O = O; p.e = e; p.a_bs = a_bs; p.w_bs = w_bs; p.o_bs = o_bs;
            return launch_gemv<EPI, NORM_NONE>(st, p, nb);
        }
        GemmTiledParams<AT, WT> p{};
        p.a = a; p.lda = lda; p.w = w; p.T = T; p.K = K; p.O = O; p.e = e; p.a_bs = a_bs; p.w_bs = w_bs; p.o_bs = o_bs;
        gemm_tiled_kernel<AT, WT, EPI><<<dim3((O + 63) / 64, (T + 63) / 64, nb), 256, 0, st>>>(p);
        return check_launch("gemm_tiled_kernel");
    }
    // rows sorted by group (expert): group z owns rows grp[z] .. grp[z+1] (device) and matrix w + z*O*K; T rows in all, no
    // group has more than max_group_rows
    template <int EPI> int matmul_grouped(cudaStream_t st, int T, int n_groups, const int* grp, int max_group_rows, const AT* a, int lda,
                                          const WT* w, const WT* w2, int K, int O, const EpiParams<AT>& e) {
        if (use_tc && dense_gemm_usable<AT, WT>(std::max(T, 2), K, O, lda)) {
            int rc = dense_gemm_launch<AT, WT, EPI>(gemm_ctx, st, T, a, lda, w, w2, K, O, e, error, grp, n_groups, max_group_rows);
            if (rc >= 0) { launches++; return rc; }
        }
        GemmTiledParams<AT, WT> p{};
        p.a = a; p.lda = lda; p.w = w; p.w2 = w2; p.T = T; p.K = K; p.O = O; p.e = e; p.grp = grp; p.w_bs = (long long)O * K;
        gemm_tiled_kernel<AT, WT, EPI><<<dim3((O + 63) / 64, (std::min(T, max_group_rows) + 63) / 64, n_groups), 256, 0, st>>>(p);
        return check_launch("gemm_tiled_kernel");
    }
    template <int EPI, int NORM> int launch_gemv(cudaStream_t st, GemvRowsParams<AT, WT> p, int nb = 1) {
        const size_t smem = ((size_t)((p.K + 3) & ~3) + 36 + 2 * 8 + 4) * 4;
        if (optin(gemv_rows_kernel<AT, WT, EPI, NORM>, smem)) return 1;
        const int rows_per_cta = EPI == EPI_GLU ? 8 : 16;
        int grid = (p.O + rows_per_cta - 1) / rows_per_cta;
        // few rows: the warps of a CTA split K instead (two row pairs per CTA)
        p.ksplit = EPI != EPI_GLU && grid < 2 * sms && p.K % Vec16<WT>::N == 0 && p.K >= 1024;
        if (p.ksplit) grid = (p.O + 3) / 4;
        p.pdl = pdl_now ? 1 : 0;
        grid = std::max(1, std::min(grid, sms * 4));
        return launch_k("gemv_rows_kernel", st, pdl_now, gemv_rows_kernel<AT, WT, EPI, NORM>, dim3(grid, nb), dim3(256), smem, p);
    }

    template <int RW, int NI> int launch_attn_t(cudaStream_t st, AttnRowsParams<AT> p, int grid_x, int grid_y) {
        // double-buffered K/V tiles when the head sizes allow 16-byte copies and two CTAs still fit an SM
        p.nbuf = (p.dk % 4 == 0 && p.dv % 4 == 0 && p.k_ld % 4 == 0 && p.v_ld % 4 == 0 && attn_smem_bytes<RW, NI>(p.dk, p.dv, 2) <= 100 * 1024) ? 2 : 1;
        const size_t smem = attn_smem_bytes<RW, NI>(p.dk, p.dv, p.nbuf);
        if (optin(attn_rows_kernel<AT, RW, NI>, smem)) return 1;
        return launch_k("attn_rows_kernel", st, pdl_now, attn_rows_kernel<AT, RW, NI>, dim3(grid_x, grid_y, p.nsplit), dim3(ATT_WARPS * 32), smem, p);
    }
    template <int RW> int launch_attn_rw(cudaStream_t st, const AttnRowsParams<AT>& p, int gx, int gy) {
        const int ni = (p.dv + 31) / 32;
        if (ni <= 1) return launch_attn_t<RW, 1>(st, p, gx, gy);
        if (ni <= 2) return launch_attn_t<RW, 2>(st, p, gx, gy);
        if (ni <= 4) return launch_attn_t<RW, 4>(st, p, gx, gy);
        return launch_attn_t<RW, 8>(st, p, gx, gy);
    }
    // attention over T query rows: the caller fills the tensors, head geometry, pitches, scale, soft-cap, window, kept first keys,
    // sink, gates and penalty;
    // the tiling, the key split of a one-row step and the merge of the splits are chosen here.  `part` is the split scratch
    // [H][MAX_SPLIT][dv + 2].  A one-row step's launches depend on pos_hint only through its 64-position bucket.
    int attention_launch(cudaStream_t st, AttnRowsParams<AT> p, float* part, uint32_t pos_hint) {
        const int kv_mul = p.H / p.G, T = p.T;
        p.part = part;
        if (p.out_ld == 0) p.out_ld = p.H * p.dv;
        if (!p.has_out_scale) p.out_scale = 1.0f;
        p.HC = std::min(kv_mul, 16);
        int tiles = (int)((pos_hint + 1 + ATT_KT - 1) / ATT_KT);
        if (p.window > 0)   // tiles a window can touch, and those of the first keys that stay visible
            tiles = std::min(tiles, (p.window + ATT_KT - 2) / ATT_KT + 1 + (p.keep_first > 0 ? (p.keep_first + ATT_KT - 1) / ATT_KT : 0));
        tiles = std::min(tiles, MAX_SPLIT);
        // a one-row step over few KV heads: fewer query heads per CTA, so that more SMs share the keys
        while (T == 1 && p.HC > 4 && p.G * ((kv_mul + p.HC - 1) / p.HC) * tiles < sms) p.HC /= 2;
        const int chunks = (kv_mul + p.HC - 1) / p.HC;
        int rw = 4;
        if (T == 1) rw = p.HC <= 4 ? 1 : (p.HC <= 8 ? 2 : 4);
        p.TQ = std::max(1, rw * ATT_WARPS / p.HC);
        p.nsplit = 1;
        if (T == 1) {   // decode: split the keys so that the GPU has enough CTAs
            p.nsplit = std::max(1, std::min({tiles, MAX_SPLIT, (2 * sms) / std::max(1, p.G * chunks)}));
        }
        const int gx = (T + p.TQ - 1) / p.TQ, gy = p.G * chunks;
        int rc = rw == 1 ? launch_attn_rw<1>(st, p, gx, gy) : (rw == 2 ? launch_attn_rw<2>(st, p, gx, gy) : launch_attn_rw<4>(st, p, gx, gy));
        if (rc) return rc;
        if (p.nsplit > 1) {
            AttnCombineParams<AT> cp{};
            cp.part = part; cp.gate = p.gate; cp.gate_logits = p.gate_logits; cp.gate_ld = p.gate_ld; cp.out = p.out; cp.rows = T * p.H; cp.H = p.H; cp.dv = p.dv; cp.nsplit = p.nsplit; cp.out_ld = p.out_ld; cp.out_scale = p.out_scale;
            return launch_k("attn_combine_kernel", st, pdl_now, attn_combine_kernel<AT>, dim3((cp.rows + 3) / 4), dim3(128), 0, cp);
        }
        return 0;
    }
    // does the attention kernel have room for these head sizes? (its K, V and probability tiles live in shared memory)
    static bool attention_fits(int dk, int dv) {
        return dv <= 256 && attn_smem_bytes<4, 8>(dk, dv, 1) - (size_t)ATT_KT * 32 * 8 * 4 + (size_t)ATT_KT * 32 * ((dv + 31) / 32) * 4 <= 227 * 1024;
    }
    // A decode step has the same launches for every position of a bucket (the key-split count of the attention is the
    // only thing that depends on the position, and it is constant over 64 positions, then fixed), and token and position
    // are read on the device: the step is captured once per bucket into a CUDA graph and replayed.  The first step of a
    // bucket runs uncaptured (it also raises the shared-memory limits of the kernels it meets).
    int decode_enqueue(cudaStream_t st, const StepParams* d_step, uint32_t pos_hint) override {
        pdl_now = use_pdl != 0;   // the embedding kernel opens the step as an ordinary launch, the rest chain on it
        const int rc = decode_enqueue_impl(st, d_step, pos_hint);
        pdl_now = false;
        return rc;
    }
    int decode_enqueue_impl(cudaStream_t st, const StepParams* d_step, uint32_t pos_hint) {
        if (pos_hint >= max_tokens) { error = "position beyond the cache (max_tokens)"; return 1; }
        if (begin_step(pos_hint, 1)) return 1;
        PosSrc ps{d_step, 0};
        const int bucket = (int)std::min<uint32_t>(pos_hint / ATT_KT + 1, (uint32_t)MAX_SPLIT);
        const uint32_t hint = bucket < MAX_SPLIT ? pos_hint : std::max<uint32_t>(pos_hint, (uint32_t)MAX_SPLIT * ATT_KT);
        if (!use_graph || keep_layers || d_step != graph_step) {
            if (d_step != graph_step) { drop_graphs(); graph_step = d_step; }
            if (!use_graph || keep_layers) {
                if (run_layers(st, 1, ps, hint)) return 1;
                return head_rows(st, 1, nullptr, d_logits);
            }
        }
        auto it = graphs.find(bucket);
        if (it == graphs.end()) {
            if (!warmed.count(bucket)) {
                warmed.insert(bucket);
                if (run_layers(st, 1, ps, hint)) return 1;
                return head_rows(st, 1, nullptr, d_logits);
            }
            const uint64_t before = launches;
            GCK(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
            int rc = run_layers(st, 1, ps, hint);
            if (!rc) rc = head_rows(st, 1, nullptr, d_logits);
            cudaGraph_t g = nullptr;
            cudaError_t ce = cudaStreamEndCapture(st, &g);
            if (rc || ce != cudaSuccess) {
                if (g) cudaGraphDestroy(g);
                if (!rc) error = std::string("cudaStreamEndCapture: ") + cudaGetErrorString(ce);
                return 1;
            }
            GraphEntry ge;
            ge.kernels = launches - before;
            launches = before;
            ce = cudaGraphInstantiate(&ge.exec, g, 0);
            cudaGraphDestroy(g);
            if (ce != cudaSuccess) { error = std::string("cudaGraphInstantiate: ") + cudaGetErrorString(ce); return 1; }
            it = graphs.emplace(bucket, ge).first;
        }
        GCK(cudaGraphLaunch(it->second.exec, st));
        launches += it->second.kernels;
        return 0;
    }
    void drop_graphs() {
        for (auto& kv : graphs) cudaGraphExecDestroy(kv.second.exec);
        graphs.clear();
        warmed.clear();
    }

    int forward_tokens(cudaStream_t st, const uint32_t* tokens, size_t n, uint32_t pos, const uint32_t* want, size_t n_want, float* d_out) override {
        if ((size_t)pos + n > max_tokens) { error = "the tokens do not fit the cache: position " + std::to_string((size_t)pos + n) + " > max_tokens " + std::to_string(max_tokens); return 1; }
        for (size_t i = 0; i < n; i++)
            if (tokens[i] >= (uint32_t)vocab) { error = "token out of range"; return 1; }
        for (size_t k = 0; k < n_want; k++)
            if (want[k] >= n) { error = "wanted row outside the step"; return 1; }
        if (n == 0) return 0;
        if (begin_step(pos, n)) return 1;
        if (ensure_scratch(std::min(n, chunk_rows))) return 1;
        if (keep_layers) {
            layer_out_rows = n <= chunk_rows ? n : 0;
            if (layer_out_rows && n_layers() * n * width > layer_out_cap) {
                dfree(d_layer_out); d_layer_out = nullptr; layer_out_cap = 0;
                if (dalloc(&d_layer_out, n_layers() * n * width)) return 1;
                layer_out_cap = n_layers() * n * width;
            }
        }
        GCK(cudaMemcpyAsync(d_tokens + pos, tokens, n * 4, cudaMemcpyHostToDevice, st));
        for (size_t c0 = 0; c0 < n; c0 += chunk_rows) {
            const int T = (int)std::min(chunk_rows, n - c0);
            PosSrc ps{nullptr, pos + (uint32_t)c0};
            if (run_layers(st, T, ps, pos + (uint32_t)c0)) return 1;
            // wanted rows of this chunk, in the order of `want`
            std::vector<uint32_t> rows, outk;
            for (size_t k = 0; k < n_want; k++)
                if (want[k] >= c0 && want[k] < c0 + (size_t)T) { rows.push_back(want[k] - (uint32_t)c0); outk.push_back((uint32_t)k); }
            if (rows.empty()) continue;
            const int m = (int)rows.size();
            bool contiguous = true;
            for (int i = 1; i < m; i++) contiguous = contiguous && outk[i] == outk[0] + (uint32_t)i;
            if (T == 1) {
                for (int i = 0; i < m; i++) if (head_rows(st, 1, nullptr, d_out + (size_t)outk[i] * vocab)) return 1;
                continue;
            }
            GCK(cudaMemcpyAsync(d_rows, rows.data(), (size_t)m * 4, cudaMemcpyHostToDevice, st));
            GCK(cudaStreamSynchronize(st));   // `rows` is a local
            if (contiguous) {
                if (head_rows(st, m, d_rows, d_out + (size_t)outk[0] * vocab)) return 1;
            } else {
                if ((size_t)m > head_tmp_rows) {
                    dfree(d_head_tmp); d_head_tmp = nullptr; head_tmp_rows = 0;
                    if (dalloc(&d_head_tmp, (size_t)m * vocab)) return 1;
                    head_tmp_rows = (size_t)m;
                }
                if (head_rows(st, m, d_rows, d_head_tmp)) return 1;
                for (int i = 0; i < m; i++)
                    GCK(cudaMemcpyAsync(d_out + (size_t)outk[i] * vocab, d_head_tmp + (size_t)i * vocab, (size_t)vocab * 4, cudaMemcpyDeviceToDevice, st));
            }
        }
        return 0;
    }

    int read_layer_outputs(cudaStream_t st, float* out, size_t capacity, size_t* n_floats) override {
        const size_t n = n_layers() * layer_out_rows * width;
        if (!keep_layers || !d_layer_out || n == 0) { error = "no layer outputs were kept"; return 1; }
        if (capacity < n) { error = "buffer too small for the layer outputs"; return 1; }
        GCK(cudaStreamSynchronize(st));
        GCK(cudaMemcpy(out, d_layer_out, n * 4, cudaMemcpyDeviceToHost));
        *n_floats = n;
        return 0;
    }
    void set_keep_layer_outputs(bool on) override { keep_layers = on; }
    void set_option(const char* name, int value) override {
        if (!strcmp(name, "chunk_rows")) chunk_rows = (size_t)std::max(1, value);
        else if (!strcmp(name, "tensor_cores")) use_tc = value;
        else if (!strcmp(name, "graphs")) { use_graph = value; if (!value) drop_graphs(); }
        else if (!strcmp(name, "pdl")) { use_pdl = value; drop_graphs(); }
        else set_model_option(name, value);
    }
    // the residual stream after layer li of the running forward_tokens call, when a test asked for it
    int keep_layer(cudaStream_t st, size_t li, int T) {
        if (keep_layers && d_layer_out && (size_t)T == layer_out_rows)
            GCK(cudaMemcpyAsync(d_layer_out + li * (size_t)T * width, x, (size_t)T * width * 4, cudaMemcpyDeviceToDevice, st));
        return 0;
    }
};

}  // namespace lmrs
