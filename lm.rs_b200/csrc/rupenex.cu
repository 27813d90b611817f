// rupenex.cu -- the Rupenex architecture (arch.h): a decoder whose sublayers read the residual stream itself and whose
// outputs are layer-normed (no bias), scaled per column and added,
//     x0 = LN(embed[token]) w;   x <- x + ls1 * LN1(mixer(x));   x <- x + ls2 * LN2(ff(x))
// with two kinds of sequence mixer, listed per layer in config.json "layers":
//   "attention"   grouped heads; q and k RMS-normed per head with one weight vector for all heads, then the first rot.dims
//                 dimensions rotated in halves (i with i + dims/2) at frequencies base^(-2i/dims) / scaling.factor; a sliding
//                 window mask.size that always keeps the first mask.keep_first positions; a learned sink per head in the
//                 softmax denominator; the concatenated heads times sigmoid(W_g x); W_o
//   "mamba2"      state-space recurrence with one decay per head: [z | x | B | C | dt] = W_in x, a short causal convolution
//                 with bias and SiLU over (x, B, C), dt = softplus(dt + dt_bias), S <- exp(-exp(A_log) dt) S + dt B x^T,
//                 y = S^T C + D x, then y silu(z) RMS-normed in norm_groups parts with a weight, W_o
// and two kinds of feed-forward: "dense" (clamped gate and up products, g sigmoid(1.702 g) (u + 1)) and "moe" (softmax
// router over experts and identity experts, choice by score + correction, weights renormalised over the chosen, experts
// W_down relu(W_up h)^2, an optional shared expert).  logits = logit_scale * head(LN(x) w).  Everything model-specific comes
// from config.json and the tensor shapes; the kernels are the generic ones of dense_ops.cuh / mixer_ops.cuh / moe_ops.cuh /
// dense_gemm.cuh, the step / chunking / graph machinery is DenseModel's.  Caches are addressed by position like those of the
// other models; the recurrent state and the convolution tails continue from the previous step and restart when a step
// begins at position 0.
#include "dense_model.cuh"
#include "mixer_ops.cuh"
#include "moe_ops.cuh"

namespace lmrs {
namespace {

enum RpMixer { RP_ATTENTION = 0, RP_SSM = 1 };
enum RpFf { RP_FF_NONE = 0, RP_FF_DENSE = 1, RP_FF_MOE = 2 };

struct RpLayerCfg {
    int kind = RP_ATTENTION;
    // attention
    int H = 0, G = 0, dk = 0, dv = 0;
    float scale = 1.0f;
    int window = 0, keep_first = 0;
    int rot_dims = 0;
    double rot_base = 10000.0, rot_factor = 1.0;
    // state-space recurrence: H heads of P = dv value channels, N state rows, G groups of B / C
    int N = 0, taps = 0, norm_groups = 1;
    // feed-forward
    int ff_kind = RP_FF_NONE;
    int ff = 0;                    // dense: hidden size; moe: hidden size of one expert
    float limit = INFINITY;
    int E = 0, I = 0, top = 0;     // experts with matrices, identity experts, choices per token
    int shared_ff = 0;
};

template <typename AT, typename WT> class RupenexModel : public DenseModel<AT, WT> {
  public:
    typedef DenseModel<AT, WT> B;
    using B::error; using B::launches; using B::info; using B::d_logits; using B::width; using B::vocab; using B::max_tokens;
    using B::sms; using B::d_tokens; using B::cap; using B::x; using B::hn; using B::d_rows; using B::MAX_SPLIT; using B::pdl_now;
    using B::dalloc; using B::dfree; using B::need; using B::upload_w; using B::upload_f32; using B::check_launch; using B::launch_k;
    using B::drop_graphs; using B::optin;

    struct Layer {
        RpLayerCfg c;
        float *norm1 = nullptr, *ls1 = nullptr, *norm2 = nullptr, *ls2 = nullptr;
        WT* w_in = nullptr; int in_rows = 0;   // fused input projection of the mixer
        WT* wo = nullptr;
        // attention
        float *qnorm = nullptr, *knorm = nullptr, *sink = nullptr, *kcache = nullptr, *vcache = nullptr;
        const float *rot_cos = nullptr, *rot_sin = nullptr;
        // state-space recurrence
        float *wconv = nullptr, *bconv = nullptr, *tail = nullptr, *dt_bias = nullptr, *a_log = nullptr, *dskip = nullptr, *onorm = nullptr,
              *state = nullptr;
        // feed-forward
        WT *wgate = nullptr, *wup = nullptr, *wdown = nullptr;   // dense: [ff][width] x2, [width][ff]; moe: [E][ff][width], [E][width][ff]
        float *router = nullptr, *correction = nullptr;
        WT *sup = nullptr, *sdown = nullptr;                      // shared expert
    };
    std::vector<Layer> layers;
    WT *embed = nullptr, *head = nullptr;
    float *embed_norm = nullptr, *final_norm = nullptr;
    float logit_scale = 1.0f;
    bool has_state = false;      // some layer carries a recurrent state
    uint32_t next_pos = 0;       // where that state stands
    // scratch for `cap` rows
    AT *h = nullptr, *att = nullptr, *act = nullptr, *xg = nullptr;
    float *proj = nullptr, *qa = nullptr, *ys = nullptr, *dtb = nullptr, *yf = nullptr, *part = nullptr, *rz = nullptr, *wts = nullptr,
          *ye = nullptr, *ysh = nullptr;
    int *eidx = nullptr, *slot = nullptr, *row_of = nullptr, *grp = nullptr;
    unsigned int* ln_counter = nullptr;   // ticket counter of the one-row products that finish with the sublayer's norm
    int max_proj = 0, max_qa = 0, max_att = 0, max_ys = 0, max_H = 0, max_dv = 0, max_act = 0, max_top = 0, max_eff = 0, max_E = 0;
    bool any_shared = false;
    int ssm_lanes = 0;   // test / measurement override of the scan's lanes per column (0: chosen by the state size)
    int ssm_cols = 0;    // ... and of its columns per thread (0: chosen by the grid size)

    size_t n_layers() const override { return layers.size(); }

    // ---- configuration ---------------------------------------------------------------------------------------------------
    int parse_layer(const Json& jl, size_t li, RpLayerCfg& c) {
        const std::string type = jl.at("type").str;
        const std::string where = "config.json layers[" + std::to_string(li) + "]";
        const Json& m = jl.at("mixer");
        c.H = (int)m.at("heads").number(0);
        c.dv = (int)m.at("vdim").number(0);
        if (type == "attention") {
            c.kind = RP_ATTENTION;
            c.G = (int)m.at("kv_heads").number(c.H);
            c.dk = (int)m.at("dim").number(0);
            if (c.dv <= 0) c.dv = c.dk;
            c.scale = (float)m.at("scale").number(1.0);
            if (m.has("mask") && m.at("mask").is_obj()) {
                c.window = (int)m.at("mask").at("size").number(0);
                c.keep_first = m.at("mask").has("keep_first") ? (int)m.at("mask").at("keep_first").number(0) : 0;
            }
            if (c.window < 0 || c.keep_first < 0) { error = where + ": mask.size and mask.keep_first must not be negative"; return 1; }
            if (m.has("rot") && m.at("rot").is_obj()) {
                const Json& r = m.at("rot");
                c.rot_dims = (int)r.at("dims").number(0);
                c.rot_base = r.at("base").number(10000.0);
                if (r.has("scaling") && r.at("scaling").is_obj()) c.rot_factor = r.at("scaling").at("factor").number(1.0);
                if (c.rot_dims < 0 || c.rot_dims > c.dk || c.rot_dims % 2 != 0) { error = where + ": rot.dims must be even and at most dim"; return 1; }
                if (c.rot_factor == 0.0) { error = where + ": rot.scaling.factor must not be zero"; return 1; }
            }
            if (c.dk <= 0 || !B::attention_fits(c.dk, c.dv)) { error = where + ": head dim " + std::to_string(c.dk) + " / vdim " + std::to_string(c.dv) + " do not fit the attention kernel's shared-memory tiles"; return 1; }
        } else if (type == "mamba2") {
            c.kind = RP_SSM;
            c.N = (int)m.at("state").number(0);
            c.G = (int)m.at("groups").number(1);
            c.taps = (int)m.at("conv").number(0);
            c.norm_groups = m.has("norm_groups") ? (int)m.at("norm_groups").number(1) : 1;
            if (c.taps < 1 || c.taps > CONV_MAX_TAPS) { error = where + ": conv must be 1 .. " + std::to_string(CONV_MAX_TAPS); return 1; }
            if (c.N <= 0 || c.N > DELTA_MAX_DK) { error = where + ": state must be 1 .. " + std::to_string(DELTA_MAX_DK); return 1; }
            if (c.norm_groups <= 0 || c.H <= 0 || c.dv <= 0 || (c.H * c.dv) % c.norm_groups != 0) { error = where + ": heads * vdim must be a multiple of norm_groups"; return 1; }
        } else { error = where + ": unknown layer type '" + type + "'"; return 1; }
        if (c.H <= 0 || c.G <= 0 || c.dv <= 0 || c.H % c.G != 0) { error = where + ": bad head geometry"; return 1; }
        if (jl.has("mlp") && jl.at("mlp").is_obj()) {
            const Json& f = jl.at("mlp");
            const std::string kind = f.has("kind") ? f.at("kind").str : "dense";
            if (kind == "dense") {
                c.ff_kind = RP_FF_DENSE;
                c.ff = (int)f.at("ff").number(0);
                if (f.has("limit")) c.limit = (float)f.at("limit").number(INFINITY);
                if (c.ff <= 0) { error = where + ": mlp.ff is required"; return 1; }
            } else if (kind == "moe") {
                c.ff_kind = RP_FF_MOE;
                c.ff = (int)f.at("expert").at("ff").number(0);
                const Json& r = f.at("router");
                c.E = (int)r.at("experts").number(0);
                c.I = r.has("identity") ? (int)r.at("identity").number(0) : 0;
                c.top = (int)r.at("top").number(0);
                if (f.has("shared") && f.at("shared").is_obj()) c.shared_ff = (int)f.at("shared").at("ff").number(0);
                if (c.E < 0 || c.I < 0 || c.E + c.I <= 0 || (c.E > 0 && c.ff <= 0) || c.top <= 0 || c.top > c.E + c.I || c.E + c.I > 4096 || c.shared_ff < 0) {
                    error = where + ": bad expert geometry";
                    return 1;
                }
            } else { error = where + ": unknown mlp kind '" + kind + "'"; return 1; }
        }
        return 0;
    }

    // ---- weights -----------------------------------------------------------------------------------------------------------
    int load_vec(const SafeTensors& st, const std::string& name, int n, float** out) {
        const StTensor* t = nullptr;
        return need(st, name, {n}, &t) || upload_f32(t, out);
    }
    int load_mat_f32(const SafeTensors& st, const std::string& name, int rows, int cols, float** out) {
        const StTensor* t = nullptr;
        return need(st, name, {rows, cols}, &t) || upload_f32(t, out);
    }
    // matrices stacked into one: rows of `parts` in order
    int load_stack(const SafeTensors& st, const std::vector<std::pair<std::string, int>>& parts, int K, WT** out, int* rows_out) {
        int rows = 0;
        for (const auto& pr : parts) rows += pr.second;
        if (dalloc(out, (size_t)rows * K)) return 1;
        int r0 = 0;
        for (const auto& pr : parts) {
            const StTensor* t = nullptr;
            if (need(st, pr.first, {pr.second, K}, &t) || upload_w(t, *out + (size_t)r0 * K)) return 1;
            r0 += pr.second;
        }
        if (rows_out) *rows_out = rows;
        return 0;
    }

    int load(const std::string& dir, const Json& cfg, const ArchOptions& opt) {
        sms = opt.sms;
        B::gemm_ctx.sms = opt.sms;
        width = (int)cfg.at("width").number(0);
        vocab = (int)cfg.at("vocab").number(0);
        if (width <= 0 || vocab <= 0) { error = "config.json: width and vocab are required"; return 1; }
        const float eps = (float)cfg.at("norm").at("eps").number(1e-6);
        logit_scale = cfg.has("logit_scale") ? (float)cfg.at("logit_scale").number(1.0) : 1.0f;
        max_tokens = opt.max_tokens ? opt.max_tokens : 4096u;
        const Json& jl = cfg.at("layers");
        if (jl.kind != Json::ARR || jl.arr.empty()) { error = "config.json: 'layers' must be a non-empty list"; return 1; }
        SafeTensors st;
        if (!st.open(dir + "/model.safetensors", error)) return 1;
        const StTensor* t = nullptr;
        if (need(st, "embed", {vocab, width}, &t) || dalloc(&embed, t->numel()) || upload_w(t, embed)) return 1;
        if (need(st, "head", {vocab, width}, &t) || dalloc(&head, t->numel()) || upload_w(t, head)) return 1;
        if (load_vec(st, "embed.norm", width, &embed_norm) || load_vec(st, "final.norm", width, &final_norm)) return 1;
        layers.resize(jl.arr.size());
        for (size_t li = 0; li < layers.size(); li++) {
            Layer& L = layers[li];
            if (parse_layer(jl.arr[li], li, L.c)) return 1;
            RpLayerCfg& c = L.c;
            const std::string p = "l" + std::to_string(li) + ".", q = p + "mix.";
            if (load_vec(st, p + "norm1", width, &L.norm1) || load_vec(st, p + "ls1", width, &L.ls1)) return 1;
            const int att_cols = c.H * c.dv;
            if (c.kind == RP_ATTENTION) {
                const int nq = c.H * c.dk, nk = c.G * c.dk, nv = c.G * c.dv;
                if (load_stack(st, {{q + "q", nq}, {q + "k", nk}, {q + "v", nv}, {q + "g", att_cols}}, width, &L.w_in, &L.in_rows)) return 1;
                if (load_vec(st, q + "q.norm", c.dk, &L.qnorm) || load_vec(st, q + "k.norm", c.dk, &L.knorm)) return 1;
                if (st.find(q + "sink") && load_vec(st, q + "sink", c.H, &L.sink)) return 1;
                if (dalloc(&L.kcache, (size_t)max_tokens * nk) || dalloc(&L.vcache, (size_t)max_tokens * nv)) return 1;
                if (c.rot_dims > 0) {
                    std::vector<double> f;
                    for (int i = 0; i < c.rot_dims / 2; i++) f.push_back(pow(c.rot_base, -2.0 * (double)i / (double)c.rot_dims) / c.rot_factor);
                    char key[160];
                    snprintf(key, sizeof key, "halves/%d/%.17g/%.17g", c.rot_dims, c.rot_base, c.rot_factor);
                    if (this->angle_tables(key, f, 1.0, &L.rot_cos, &L.rot_sin)) return 1;
                }
                max_qa = std::max(max_qa, nq);
            } else {
                const int inner = att_cols, gn = c.G * c.N, C = inner + 2 * gn;
                if (load_stack(st, {{q + "in", 2 * inner + 2 * gn + c.H}}, width, &L.w_in, &L.in_rows)) return 1;
                if (load_mat_f32(st, q + "conv", C, c.taps, &L.wconv)) return 1;
                if (st.find(q + "conv.b") && load_vec(st, q + "conv.b", C, &L.bconv)) return 1;
                if (load_vec(st, q + "dt_bias", c.H, &L.dt_bias) || load_vec(st, q + "A_log", c.H, &L.a_log) || load_vec(st, q + "norm", inner, &L.onorm)) return 1;
                if (st.find(q + "D") && load_vec(st, q + "D", c.H, &L.dskip)) return 1;
                if (dalloc(&L.state, (size_t)c.H * c.N * c.dv) || dalloc(&L.tail, (size_t)std::max(c.taps - 1, 1) * C)) return 1;
                GCK(cudaMemset(L.state, 0, (size_t)c.H * c.N * c.dv * 4));
                GCK(cudaMemset(L.tail, 0, (size_t)std::max(c.taps - 1, 1) * C * 4));
                has_state = true;
                max_qa = std::max(max_qa, C);
                max_ys = std::max(max_ys, inner);
            }
            if (load_stack(st, {{q + "o", width}}, att_cols, &L.wo, nullptr)) return 1;
            max_proj = std::max(max_proj, L.in_rows);
            max_att = std::max(max_att, att_cols);
            max_H = std::max(max_H, c.H);
            max_dv = std::max(max_dv, c.dv);
            if (c.ff_kind != RP_FF_NONE && (load_vec(st, p + "norm2", width, &L.norm2) || load_vec(st, p + "ls2", width, &L.ls2))) return 1;
            if (c.ff_kind == RP_FF_DENSE) {
                if (load_stack(st, {{p + "mlp.gate", c.ff}}, width, &L.wgate, nullptr) || load_stack(st, {{p + "mlp.up", c.ff}}, width, &L.wup, nullptr) ||
                    load_stack(st, {{p + "mlp.down", width}}, c.ff, &L.wdown, nullptr))
                    return 1;
                max_act = std::max(max_act, c.ff);
            } else if (c.ff_kind == RP_FF_MOE) {
                const int n = c.E + c.I;
                if (load_mat_f32(st, p + "mlp.router", n, width, &L.router)) return 1;
                if (st.find(p + "mlp.correction") && load_vec(st, p + "mlp.correction", n, &L.correction)) return 1;
                std::vector<std::pair<std::string, int>> us, ds;
                for (int e = 0; e < c.E; e++) {
                    const std::string pe = p + "mlp.e" + std::to_string(e) + ".";
                    us.push_back({pe + "up", c.ff}); ds.push_back({pe + "down", width});
                }
                if (c.E > 0 && (load_stack(st, us, width, &L.wup, nullptr) || load_stack(st, ds, c.ff, &L.wdown, nullptr))) return 1;
                if (c.shared_ff > 0) {
                    if (load_stack(st, {{p + "mlp.shared.up", c.shared_ff}}, width, &L.sup, nullptr) ||
                        load_stack(st, {{p + "mlp.shared.down", width}}, c.shared_ff, &L.sdown, nullptr))
                        return 1;
                    any_shared = true;
                    max_act = std::max(max_act, c.shared_ff);
                }
                max_top = std::max(max_top, c.top); max_eff = std::max(max_eff, c.ff); max_E = std::max(max_E, n);
            }
        }
        if (dalloc(&d_tokens, (size_t)max_tokens) || dalloc(&d_logits, (size_t)vocab) || dalloc(&ln_counter, 1)) return 1;
        GCK(cudaMemset(d_tokens, 0, (size_t)max_tokens * 4));
        GCK(cudaMemset(ln_counter, 0, sizeof(unsigned int)));
        info.architecture = "Rupenex";
        info.model_type = 5;
        info.vocab = (uint32_t)vocab; info.width = (uint32_t)width; info.n_layers = (uint32_t)layers.size(); info.max_tokens = max_tokens;
        info.heads = (uint32_t)layers[0].c.H; info.kv_heads = (uint32_t)layers[0].c.G; info.head_dim = (uint32_t)(layers[0].c.kind == RP_ATTENTION ? layers[0].c.dk : layers[0].c.dv);
        info.ff = (uint32_t)layers[0].c.ff; info.dtype = opt.dtype; info.eps = eps;
        return ensure_scratch(1);
    }

    int ensure_scratch(size_t rows) override {
        if (rows <= cap) return 0;
        drop_graphs();   // captured launches point into the old scratch
        for (void* p : {(void*)x, (void*)hn, (void*)d_rows, (void*)h, (void*)att, (void*)act, (void*)xg, (void*)proj, (void*)qa, (void*)ys, (void*)dtb,
                        (void*)yf, (void*)part, (void*)rz, (void*)wts, (void*)ye, (void*)ysh, (void*)eidx, (void*)slot, (void*)row_of, (void*)grp})
            dfree(p);
        cap = 0;
        const size_t pairs = rows * std::max(max_top, 1);
        const size_t act_n = std::max(rows * (size_t)std::max(max_act, 1), pairs * (size_t)std::max(max_eff, 1));
        if (dalloc(&x, rows * width) || dalloc(&hn, rows * width) || dalloc(&d_rows, rows) || dalloc(&h, rows * width) || dalloc(&att, rows * max_att) ||
            dalloc(&act, act_n) || dalloc(&proj, rows * max_proj) || dalloc(&qa, rows * max_qa) || dalloc(&ys, rows * std::max(max_ys, 1)) ||
            dalloc(&dtb, rows * 2 * max_H) || dalloc(&yf, rows * width) || dalloc(&part, (size_t)max_H * MAX_SPLIT * (max_dv + 2)))
            return 1;
        if (max_top > 0 &&
            (dalloc(&xg, pairs * width) || dalloc(&rz, rows * max_E) || dalloc(&wts, pairs) || dalloc(&ye, pairs * width) || dalloc(&eidx, pairs) ||
             dalloc(&slot, pairs) || dalloc(&row_of, pairs) || dalloc(&grp, (size_t)max_E + 1)))
            return 1;
        if (any_shared && dalloc(&ysh, rows * width)) return 1;
        cap = rows;
        return 0;
    }

    // the recurrent state stands at one position: a step continues there or starts a new sequence at 0
    int begin_step(uint32_t pos, size_t n) override {
        if (!has_state) return 0;
        if (pos != 0 && pos != next_pos) {
            error = "a model with recurrent layers continues at position " + std::to_string(next_pos) + " or restarts at 0, not at " + std::to_string(pos);
            return 1;
        }
        next_pos = pos + (uint32_t)n;
        return 0;
    }

    // ---- the layers -----------------------------------------------------------------------------------------------------------
    // v = LN(in) w;  with ls: x <- x + ls * v, and x's rows again in the operand type (h) for the next matrix product
    int norm_into_residual(cudaStream_t st, int T, const float* in, const float* w, const float* ls) {
        LayerNormRowsParams<AT> p{};
        p.in = in; p.ld_in = width; p.w = w; p.eps = info.eps; p.n = width;
        if (ls) { p.resid = x; p.ld_resid = width; p.ls = ls; }
        else { p.out_f = x; p.ld_f = width; }
        p.out_op = h; p.ldo = width;
        return launch_k("layernorm_rows_kernel", st, pdl_now, layernorm_rows_kernel<AT>, dim3(T), dim3(256), 0, p);
    }
    // yf = a . wo^T, then into the residual stream through the sublayer's norm
    // (one row: the product's last CTA applies the norm itself)
    int out_proj(cudaStream_t st, int T, const AT* a, int K, const WT* wo, const float* nw, const float* ls) {
        EpiParams<AT> e{}; e.out = yf; e.ldo = width; e.scale = 1.0f;
        if (T == 1) {
            GemvRowsParams<AT, WT> p{};
            p.a = a; p.w = wo; p.K = K; p.O = width; p.e = e;
            p.ln.counter = ln_counter; p.ln.w = nw; p.ln.ls = ls; p.ln.eps = info.eps; p.ln.x = x; p.ln.h = h;
            return this->template launch_gemv<EPI_STORE, NORM_NONE>(st, p);
        }
        if (this->template matmul<EPI_STORE>(st, T, a, K, wo, nullptr, K, width, e)) return 1;
        return norm_into_residual(st, T, yf, nw, ls);
    }
    int in_proj(cudaStream_t st, const Layer& L, int T) {
        EpiParams<AT> e{}; e.out = proj; e.ldo = L.in_rows; e.scale = 1.0f;
        return this->template matmul<EPI_STORE>(st, T, h, width, L.w_in, nullptr, width, L.in_rows, e);
    }

    int mixer_attention(cudaStream_t st, const Layer& L, int T, const PosSrc& ps, uint32_t pos_hint) {
        const RpLayerCfg& c = L.c;
        if (in_proj(st, L, T)) return 1;
        QkvPostParams qp{};
        qp.qkv = proj; qp.ld = L.in_rows; qp.H = c.H; qp.G = c.G; qp.dk = c.dk; qp.dv = c.dv;
        qp.qk_mode = c.rot_dims > 0 ? QK_ROTARY : QK_PLAIN; qp.eps = info.eps; qp.q_nw = L.qnorm; qp.k_nw = L.knorm;
        qp.rot_dims = c.rot_dims; qp.rot_cos = L.rot_cos; qp.rot_sin = L.rot_sin;
        qp.v_mode = V_PLAIN; qp.has_gate = false; qp.q_out = qa; qp.kcache = L.kcache; qp.vcache = L.vcache; qp.ps = ps;
        const int tasks = c.H + c.G + (c.G * c.dv + 127) / 128;
        const dim3 grid(T, T >= 64 ? std::min(4, (tasks + 3) / 4) : std::min(16, (tasks + 3) / 4));
        if (launch_k("qkv_post_kernel", st, pdl_now, qkv_post_kernel, grid, dim3(128), 0, qp)) return 1;
        AttnRowsParams<AT> p{};
        p.q = qa; p.kcache = L.kcache; p.vcache = L.vcache; p.out = att;
        p.T = T; p.H = c.H; p.G = c.G; p.dk = c.dk; p.dv = c.dv; p.scale = c.scale; p.ps = ps;
        p.k_ld = c.G * c.dk; p.v_ld = c.G * c.dv; p.window = c.window; p.keep_first = c.keep_first; p.sink = L.sink;
        p.gate_logits = proj + (size_t)(c.H + c.G) * c.dk + (size_t)c.G * c.dv; p.gate_ld = L.in_rows;
        if (this->attention_launch(st, p, part, pos_hint)) return 1;
        return out_proj(st, T, att, c.H * c.dv, L.wo, L.norm1, L.ls1);
    }

    template <int NR, int LPC, int CPT> int launch_scan(cudaStream_t st, const SsmScanParams& sp) {
        constexpr int cols = DELTA_THREADS / LPC * CPT;
        const size_t smem = ssm_scan_smem(NR, LPC, CPT);
        if (optin(ssm_scan_kernel<NR, LPC, CPT>, smem)) return 1;
        return launch_k("ssm_scan_kernel", st, pdl_now, ssm_scan_kernel<NR, LPC, CPT>, dim3((sp.P + cols - 1) / cols, sp.H), dim3(DELTA_THREADS), smem, sp);
    }
    int mixer_ssm(cudaStream_t st, const Layer& L, int T, const PosSrc& ps) {
        const RpLayerCfg& c = L.c;
        const int inner = c.H * c.dv, gn = c.G * c.N, C = inner + 2 * gn;
        if (in_proj(st, L, T)) return 1;
        float* dt = dtb;
        float* decay = dtb + (size_t)cap * c.H;
        SsmPreParams pp{};
        pp.in = proj; pp.ld = L.in_rows; pp.c_off = inner; pp.C = C; pp.taps = c.taps; pp.wconv = L.wconv; pp.bconv = L.bconv; pp.tail = L.tail;
        pp.out = qa; pp.dt_off = 2 * inner + 2 * gn; pp.H = c.H; pp.dt_bias = L.dt_bias; pp.a_log = L.a_log; pp.dt = dt; pp.decay = decay; pp.T = T; pp.ps = ps;
        const bool tail_here = c.taps > 1 && T <= SSM_PRE_TT;   // one block of tokens: its threads move the tail on themselves
        if (tail_here) pp.tail_out = L.tail;
        if (launch_k("ssm_pre_kernel", st, pdl_now, ssm_pre_kernel, dim3((C + 127) / 128 + 1, (T + SSM_PRE_TT - 1) / SSM_PRE_TT), dim3(128), 0, pp)) return 1;
        if (c.taps > 1 && !tail_here) {
            ConvTailParams tp{};
            tp.in = proj + inner; tp.ld = L.in_rows; tp.tail = L.tail; tp.C = C; tp.taps = c.taps; tp.T = T; tp.ps = ps;
            if (launch_k("conv_tail_update_kernel", st, pdl_now, conv_tail_update_kernel, dim3((C + 255) / 256), dim3(256), 0, tp)) return 1;
        }
        SsmScanParams sp{};
        sp.xbc = qa; sp.ld = C; sp.b_off = inner; sp.c_off = inner + gn; sp.dt = dt; sp.decay = decay; sp.D = L.dskip; sp.state = L.state; sp.out = ys;
        sp.T = T; sp.H = c.H; sp.G = c.G; sp.N = c.N; sp.P = c.dv; sp.ps = ps;
        // (rows per lane, lanes per column) with rows * lanes >= N.  The read-out's lane reduction is not on the path to the next
        // token's state (unlike the delta rule's), so fewer lanes with more rows each do better here: 8 lanes of 16 rows at 128
        // state rows measured 5 % under 16 lanes of 8, and 4 lanes of 32 another 1 % at half as many CTAs
        int lpc = ssm_lanes > 0 ? ssm_lanes : (c.N <= 16 ? 1 : c.N <= 32 ? 2 : c.N <= 64 ? 4 : c.N <= 128 ? 8 : c.N <= 256 ? 16 : 32);
        while (lpc < 32 && 32 * lpc < c.N) lpc *= 2;
        const int nr = 8 * lpc >= c.N ? 8 : (16 * lpc >= c.N ? 16 : 32);
        int rc = 1;
#define RP_SCAN(NR_, LPC_) if (nr == NR_ && lpc == LPC_) rc = launch_scan<NR_, LPC_, 1>(st, sp); else
        // two columns per thread share each read of a token's B and C entries (12 % off the scan at 64 heads of 64 x 128); taken
        // when the grid still has a CTA for at least half of the SMs
        const bool two_ok = (nr == 8 && (lpc == 8 || lpc == 16)) || (nr == 16 && lpc == 8);
        const int ctas2 = ((c.dv + 2 * (DELTA_THREADS / lpc) - 1) / (2 * (DELTA_THREADS / lpc))) * c.H;
        const int cpt = ssm_cols > 0 ? ssm_cols : (two_ok && 2 * ctas2 >= sms ? 2 : 1);
        if (cpt == 2 && nr == 8 && lpc == 16) rc = launch_scan<8, 16, 2>(st, sp);
        else if (cpt == 2 && nr == 16 && lpc == 8) rc = launch_scan<16, 8, 2>(st, sp);
        else if (cpt == 2 && nr == 8 && lpc == 8) rc = launch_scan<8, 8, 2>(st, sp);
        else
        RP_SCAN(8, 1) RP_SCAN(16, 1) RP_SCAN(8, 2) RP_SCAN(16, 2) RP_SCAN(32, 2) RP_SCAN(8, 4) RP_SCAN(16, 4) RP_SCAN(32, 4) RP_SCAN(8, 8) RP_SCAN(16, 8)
        RP_SCAN(32, 8) RP_SCAN(8, 16) RP_SCAN(16, 16) RP_SCAN(32, 16) RP_SCAN(8, 32) RP_SCAN(16, 32) { error = "no scan kernel for state " + std::to_string(c.N); return 1; }
#undef RP_SCAN
        if (rc) return 1;
        GatedGroupNormParams<AT> gp{};
        gp.y = ys; gp.ldy = inner; gp.z = proj; gp.ldz = L.in_rows; gp.w = L.onorm; gp.eps = info.eps; gp.out = att; gp.ldo = inner; gp.n = inner; gp.groups = c.norm_groups;
        if (launch_k("gated_groupnorm_kernel", st, pdl_now, gated_groupnorm_kernel<AT>, dim3(T, c.norm_groups), dim3(256), 0, gp)) return 1;
        return out_proj(st, T, att, inner, L.wo, L.norm1, L.ls1);
    }

    int ff_dense(cudaStream_t st, const Layer& L, int T) {
        const RpLayerCfg& c = L.c;
        EpiParams<AT> eg{}; eg.act = act; eg.lda = c.ff; eg.glu_kind = GLU_CLAMPED; eg.glu_limit = c.limit; eg.glu_alpha = 1.702f;
        if (this->template matmul<EPI_GLU>(st, T, h, width, L.wgate, L.wup, width, c.ff, eg)) return 1;
        return out_proj(st, T, act, c.ff, L.wdown, L.norm2, L.ls2);
    }

    int ff_moe(cudaStream_t st, const Layer& L, int T) {
        const RpLayerCfg& c = L.c;
        const int n_out = c.E + c.I;
        MoeRouterParams<AT> rp{};
        rp.h = h; rp.ld = width; rp.router = L.router; rp.correction = L.correction; rp.E = n_out; rp.top = c.top; rp.width = width; rp.softmax = 1;
        rp.scale = 1.0f; rp.z = rz; rp.idx = eidx; rp.wts = wts;
        if (launch_k("moe_logits_kernel", st, pdl_now, moe_logits_kernel<AT>, dim3(T, (n_out + 3) / 4), dim3(128), 0, rp)) return 1;
        if (launch_k("moe_topk_kernel", st, pdl_now, moe_topk_kernel<AT>, dim3(T), dim3(32), (size_t)2 * n_out * 4, rp)) return 1;
        MoeCombineParams cp{};
        cp.y = ye; cp.wts = wts; cp.top = c.top; cp.width = width; cp.idx = eidx; cp.n_real = c.E; cp.xin = x; cp.ld_in = width; cp.x = x; cp.ldx = width;
        EpiParams<AT> eu{}; eu.act = act; eu.lda = c.ff; eu.act_kind = ACT_RELU2;
        EpiParams<AT> ed{}; ed.out = ye; ed.ldo = width; ed.scale = 1.0f;
        if (c.E > 0) {
            if (T == 1) {   // the chosen experts' matrices, picked on the device from the router's list; identity experts have none
                GemvRowsParams<AT, WT> u{};
                u.a = h; u.w = L.wup; u.K = width; u.O = c.ff; u.e = eu; u.bidx = eidx; u.w_bs = (long long)c.ff * width; u.o_bs = c.ff; u.n_mats = c.E;
                if (this->template launch_gemv<EPI_ACT, NORM_NONE>(st, u, c.top)) return 1;
                GemvRowsParams<AT, WT> d{};
                d.a = act; d.w = L.wdown; d.K = c.ff; d.O = width; d.e = ed; d.bidx = eidx; d.a_bs = c.ff; d.w_bs = (long long)width * c.ff; d.o_bs = width; d.n_mats = c.E;
                if (this->template launch_gemv<EPI_STORE, NORM_NONE>(st, d, c.top)) return 1;
                cp.slot = nullptr;
            } else {   // rows sorted by expert; identity experts sort behind the experts with matrices and take no product
                const int n = T * c.top;
                MoeSortParams sp{};
                sp.idx = eidx; sp.n = n; sp.E = n_out; sp.top = c.top; sp.grp = grp; sp.slot = slot; sp.row_of = row_of;
                if (launch_k("moe_sort_kernel", st, pdl_now, moe_sort_kernel, dim3(1), dim3(1024), (size_t)2 * n_out * 4, sp)) return 1;
                MoeGatherParams<AT> gp{};
                gp.h = h; gp.ld = width; gp.row_of = row_of; gp.out = xg; gp.width = width;
                if (launch_k("moe_gather_kernel", st, pdl_now, moe_gather_kernel<AT>, dim3(n), dim3(128), 0, gp)) return 1;
                if (this->template matmul_grouped<EPI_ACT>(st, n, c.E, grp, T, xg, width, L.wup, nullptr, width, c.ff, eu)) return 1;
                if (this->template matmul_grouped<EPI_STORE>(st, n, c.E, grp, T, act, c.ff, L.wdown, nullptr, c.ff, width, ed)) return 1;
                cp.slot = slot;
            }
        }
        if (c.shared_ff > 0) {
            EpiParams<AT> su{}; su.act = act; su.lda = c.shared_ff; su.act_kind = ACT_RELU2;
            if (this->template matmul<EPI_ACT>(st, T, h, width, L.sup, nullptr, width, c.shared_ff, su)) return 1;
            EpiParams<AT> sd{}; sd.out = ysh; sd.ldo = width; sd.scale = 1.0f;
            if (this->template matmul<EPI_STORE>(st, T, act, c.shared_ff, L.sdown, nullptr, c.shared_ff, width, sd)) return 1;
            cp.add = ysh;
        }
        MoeCombineNormParams<AT> np{};
        np.c = cp; np.w = L.norm2; np.ls = L.ls2; np.eps = info.eps; np.h = h; np.ldh = width; np.counter = ln_counter;
        if (T == 1) { np.c.out = yf; np.c.ldo = width; }   // one row: its columns spread over several CTAs, the last one norms
        return launch_k("moe_combine_layernorm_kernel", st, pdl_now, moe_combine_layernorm_kernel<AT>, dim3(T, T == 1 ? (width + 255) / 256 : 1), dim3(256), 0, np);
    }

    int run_layers(cudaStream_t st, int T, const PosSrc& ps, uint32_t pos_hint) override {
        {
            EmbedRowsParams<WT> p{};
            p.embed = embed; p.bigram = nullptr; p.tokens = d_tokens; p.x = x; p.width = width; p.ps = ps;
            embed_rows_kernel<WT><<<T, 128, 0, st>>>(p);
            if (check_launch("embed_rows_kernel")) return 1;
            if (norm_into_residual(st, T, x, embed_norm, nullptr)) return 1;
        }
        for (size_t li = 0; li < layers.size(); li++) {
            const Layer& L = layers[li];
            if (L.c.kind == RP_ATTENTION ? mixer_attention(st, L, T, ps, pos_hint) : mixer_ssm(st, L, T, ps)) return 1;
            if (L.c.ff_kind == RP_FF_DENSE && ff_dense(st, L, T)) return 1;
            if (L.c.ff_kind == RP_FF_MOE && ff_moe(st, L, T)) return 1;
            if (this->keep_layer(st, li, T)) return 1;
        }
        return 0;
    }
    int head_rows(cudaStream_t st, int m, const uint32_t* rows_dev, float* out) override {
        EpiParams<AT> e{}; e.out = out; e.ldo = vocab; e.scale = logit_scale;
        if (m == 1 && rows_dev == nullptr) {
            GemvRowsParams<AT, WT> p{};
            p.x = x; p.nw = final_norm; p.eps = info.eps; p.w = head; p.K = width; p.O = vocab; p.e = e;
            return this->template launch_gemv<EPI_STORE, NORM_LAYER>(st, p);
        }
        LayerNormRowsParams<AT> np{};
        np.in = x; np.ld_in = width; np.rows = rows_dev; np.w = final_norm; np.eps = info.eps; np.n = width; np.out_op = hn; np.ldo = width;
        if (launch_k("layernorm_rows_kernel", st, pdl_now, layernorm_rows_kernel<AT>, dim3(m), dim3(256), 0, np)) return 1;
        return this->template matmul<EPI_STORE>(st, m, hn, width, head, nullptr, width, vocab, e);
    }

    void set_model_option(const char* name, int value) override {
        if (!strcmp(name, "ssm_lanes")) { ssm_lanes = value; drop_graphs(); }
        if (!strcmp(name, "ssm_cols")) { ssm_cols = value; drop_graphs(); }
    }
    // test access: K and V rows of an attention layer; a state-space layer keeps a state, not rows per position
    int read_kv(cudaStream_t st, uint32_t layer, uint32_t pos0, uint32_t n, float* k_out, float* v_out) override {
        if (layer >= layers.size() || (size_t)pos0 + n > max_tokens) { error = "read_kv: out of range"; return 1; }
        const Layer& L = layers[layer];
        if (L.c.kind != RP_ATTENTION) { error = "read_kv: a state-space layer keeps a state, not rows per position"; return 1; }
        GCK(cudaStreamSynchronize(st));
        const size_t nk = (size_t)L.c.G * L.c.dk, nv = (size_t)L.c.G * L.c.dv;
        GCK(cudaMemcpy(k_out, L.kcache + pos0 * nk, n * nk * 4, cudaMemcpyDeviceToHost));
        GCK(cudaMemcpy(v_out, L.vcache + pos0 * nv, n * nv * 4, cudaMemcpyDeviceToHost));
        return 0;
    }
};

ArchModel* rupenex_factory(const std::string& dir, const Json& cfg, const ArchOptions& opt, std::string& err) {
    ArchModel* m = nullptr;
    int rc;
    if (opt.dtype == ARCH_F32) {
        auto* g = new RupenexModel<float, float>();
        rc = g->load(dir, cfg, opt);
        m = g;
    } else {
        auto* g = new RupenexModel<__nv_bfloat16, __nv_bfloat16>();
        rc = g->load(dir, cfg, opt);
        m = g;
    }
    if (rc) { err = m->error; delete m; return nullptr; }
    return m;
}

}  // namespace

void register_rupenex() { arch_register("Rupenex", rupenex_factory); }

}  // namespace lmrs
