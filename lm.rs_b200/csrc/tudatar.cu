// tudatar.cu -- the Tudatar architecture (arch.h): a decoder whose layers are SEQUENTIAL blocks with a norm before and after
// each sublayer,
//     x <- x + N1b(mixer(N1(x)));   x <- x + N2b(ff(N2(x)))        N(v) = tanh(alpha v) w + b   (no statistics)
// with three kinds of sequence mixer, listed per layer in config.json "layers":
//   "channel_delta"     gated delta rule: short causal convolution + SiLU on q, k, v, unit-length q and k, one decay per head
//                       and key channel from a low-rank projection, state S [dk][dv] per head in f32, output RMS-normed per
//                       head and gated by a second low-rank projection
//   "latent_attention"  softmax attention whose keys and values are up-projections of one cached latent per token plus one
//                       rotated key part shared by all heads; queries go through a latent of their own.  Short steps run in
//                       the latent space: the up-projection of the keys is multiplied into the query, the attention kernel
//                       sees one shared key/value head of size kv_rank (+ rot_dim), and the values' up-projection follows it.
//                       Long portions up-project all cached latents to per-head keys and values first (tensor cores) and run
//                       ordinary multi-head attention over them: a third of the attention arithmetic
//   "attention"         grouped-head attention with projection biases, q and k RMS-normed over the whole projection, values
//                       normed per head, a sliding window and a logarithmic distance penalty per head, no rotation
// and a feed-forward of routed experts (sigmoid router, choice with a correction, normalised weights).  logits =
// logit_scale * head(N_final(x)).  Everything model-specific comes from config.json and the tensor shapes; the kernels are
// the generic ones of dense_ops.cuh / mixer_ops.cuh / moe_ops.cuh / dense_gemm.cuh, the step / chunking / graph machinery
// is DenseModel's.  Caches are addressed by position like those of the other models; the recurrent state and the convolution
// tails continue from the previous step and restart when a step begins at position 0.
#include "dense_model.cuh"
#include "mixer_ops.cuh"
#include "moe_ops.cuh"

namespace lmrs {
namespace {

enum MixerKind { MIX_DELTA = 0, MIX_LATENT = 1, MIX_WINDOW = 2 };

struct RotSpec {   // pairwise rotation with frequencies rescaled between two wavelengths
    int dims = 0;
    double base = 10000.0;
    bool scaled = false;
    double factor = 1.0, fast = 32.0, slow = 1.0, original = 1.0;
    std::string key() const {
        char b[256];
        snprintf(b, sizeof b, "pairs/%d/%.17g/%d/%.17g/%.17g/%.17g/%.17g", dims, base, (int)scaled, factor, fast, slow, original);
        return b;
    }
    // frequencies f_i and the multiplier of cos and sin
    void freqs(std::vector<double>& f, double& mult) const {
        const double kPi = 3.14159265358979323846;
        f.clear();
        mult = 1.0;
        for (int i = 0; i < dims / 2; i++) f.push_back(pow(base, -2.0 * (double)i / (double)dims));
        if (!scaled) return;
        // the (fractional) pair index whose wavelength makes `turns` turns over the original length
        auto where = [&](double turns) { return (double)dims * log(original / (2.0 * kPi * turns)) / (2.0 * log(base)); };
        const double lo = std::max(floor(where(fast)), 0.0), hi = std::min(ceil(where(slow)), (double)dims - 1.0);
        for (int i = 0; i < dims / 2; i++) {
            const double ramp = std::min(1.0, std::max(0.0, ((double)i - lo) / std::max(hi - lo, 0.001)));
            f[i] = f[i] / factor * ramp + f[i] * (1.0 - ramp);
        }
        mult = 0.1 * log(factor) + 1.0;
    }
};
struct MoeCfg {
    bool on = false;
    int E = 0, top = 0, ff = 0;
    float scale = 1.0f;
};
struct LayerCfg {
    int kind = MIX_WINDOW;
    int H = 0, G = 0, dk = 0, dv = 0;
    float scale = 1.0f;
    int window = 0;                       // MIX_WINDOW
    int taps = 0, ra = 0, rg = 0;         // MIX_DELTA
    int dr = 0, rk = 0, rq = 0;           // MIX_LATENT (dk = unrotated size)
    bool latent_space_ok = true, per_head_ok = true;
    RotSpec rot;
    MoeCfg moe;
};

template <typename AT, typename WT> class TudatarModel : public DenseModel<AT, WT> {
  public:
    typedef DenseModel<AT, WT> B;
    using B::error; using B::launches; using B::info; using B::d_logits; using B::width; using B::vocab; using B::max_tokens;
    using B::sms; using B::d_tokens; using B::cap; using B::x; using B::hn; using B::d_rows; using B::MAX_SPLIT; using B::pdl_now;
    using B::dalloc; using B::dfree; using B::need; using B::upload_w; using B::upload_f32; using B::check_launch; using B::launch_k;
    using B::drop_graphs; using B::optin;

    struct Norm { float *alpha = nullptr, *w = nullptr, *b = nullptr; TanhNorm view() const { return TanhNorm{alpha, w, b}; } };
    struct Layer {
        LayerCfg c;
        Norm n1, n1b, n2, n2b;
        WT* w_in = nullptr; int in_rows = 0;    // fused input projection of the mixer
        float* b_in = nullptr;                   // its bias (MIX_WINDOW)
        WT* wo = nullptr;
        // MIX_WINDOW
        float *qnorm = nullptr, *knorm = nullptr, *r1 = nullptr, *r2 = nullptr, *kcache = nullptr, *vcache = nullptr;
        // MIX_LATENT
        float *dq_norm = nullptr, *dkv_norm = nullptr, *lcache = nullptr;
        AT* lcache_op = nullptr;                               // [max_tokens][rk] the latent in the operand type
        WT *wuq = nullptr, *wuk = nullptr, *wukT = nullptr, *wuv = nullptr;   // wukT: [H][rk][dn], wuk transposed per head
        const float *rot_cos = nullptr, *rot_sin = nullptr;
        // MIX_DELTA
        float *wconv = nullptr, *tail = nullptr, *a_log = nullptr, *onorm = nullptr, *dt_bias = nullptr, *state = nullptr;
        WT *wa2 = nullptr, *wg2 = nullptr;
        // routed experts
        float *router = nullptr, *correction = nullptr;
        WT *wgate = nullptr, *wup = nullptr, *wdown = nullptr;   // [E][ff][width], [E][ff][width], [E][width][ff]
    };
    std::vector<Layer> layers;
    WT *embed = nullptr, *head = nullptr;
    Norm final_norm;
    float logit_scale = 1.0f;
    bool has_state = false;      // some layer carries a recurrent state
    uint32_t next_pos = 0;       // where that state stands
    // scratch for `cap` rows
    AT *h = nullptr, *lat = nullptr, *qn = nullptr, *att = nullptr, *att2 = nullptr, *xg = nullptr, *act = nullptr;
    float *rz = nullptr, *proj = nullptr, *qa = nullptr, *qb = nullptr, *fa = nullptr, *fb = nullptr, *beta = nullptr, *part = nullptr, *y = nullptr, *wts = nullptr;
    int *eidx = nullptr, *slot = nullptr, *row_of = nullptr, *grp = nullptr;
    float *kfull = nullptr, *vfull = nullptr, *knope = nullptr;   // per-head keys and values of all cached positions (long latent-attention portions)
    int max_kfull = 0, max_vfull = 0, max_knope = 0;
    int latent_expand_rows = 16;   // portions of at least this many rows take the per-head form
    int max_proj = 0, max_lat = 0, max_qn = 0, max_att = 0, max_att2 = 0, max_qa = 0, max_qb = 0, max_fa = 0, max_fb = 0, max_H = 0,
        max_dv = 0, max_top = 0, max_ff = 0, max_E = 0;

    size_t n_layers() const override { return layers.size(); }

    // ---- configuration ---------------------------------------------------------------------------------------------------
    int parse_layer(const Json& jl, size_t li, LayerCfg& c) {
        const std::string type = jl.at("type").str;
        const std::string where = "config.json layers[" + std::to_string(li) + "]";
        const Json& m = jl.at("mixer");
        c.H = (int)m.at("heads").number(0);
        c.dk = (int)m.at("dim").number(0);
        c.dv = (int)m.at("vdim").number(c.dk);
        if (type == "channel_delta") {
            c.kind = MIX_DELTA;
            c.G = (int)m.at("kv_heads").number(c.H);
            c.taps = (int)m.at("conv").number(0);
            if (c.taps < 1 || c.taps > CONV_MAX_TAPS) { error = where + ": conv must be 1 .. " + std::to_string(CONV_MAX_TAPS); return 1; }
            if (c.dk > DELTA_MAX_DK) { error = where + ": dim above " + std::to_string(DELTA_MAX_DK) + " is not supported by the delta-rule kernel"; return 1; }
        } else if (type == "latent_attention") {
            c.kind = MIX_LATENT;
            c.G = 1;
            c.dr = (int)m.at("rot_dim").number(0); c.rk = (int)m.at("kv_rank").number(0); c.rq = (int)m.at("q_rank").number(0);
            c.scale = (float)m.at("scale").number(1.0);
            if (c.dr < 0 || c.rk <= 0 || c.rq <= 0) { error = where + ": rot_dim, kv_rank and q_rank are required"; return 1; }
            const Json& r = m.at("rot");
            c.rot.dims = r.is_obj() ? (int)r.at("dims").number(c.dr) : 0;
            if (c.rot.dims < 0 || c.rot.dims > c.dr || c.rot.dims % 2 != 0) { error = where + ": rot.dims must be even and at most rot_dim"; return 1; }
            if (r.is_obj()) {
                c.rot.base = r.at("base").number(10000.0);
                if (r.has("scaling") && r.at("scaling").is_obj()) {
                    const Json& s = r.at("scaling");
                    c.rot.scaled = true;
                    c.rot.factor = s.at("factor").number(1.0); c.rot.fast = s.at("fast").number(32.0);
                    c.rot.slow = s.at("slow").number(1.0); c.rot.original = s.at("original").number(4096.0);
                }
            }
            // a latent too wide for the attention kernel's tiles is always up-projected to per-head keys and values
            c.latent_space_ok = B::attention_fits(c.rk + c.dr, c.rk);
            c.per_head_ok = B::attention_fits(c.dk + c.dr, c.dv);
            if (!c.latent_space_ok && !c.per_head_ok) { error = where + ": neither kv_rank " + std::to_string(c.rk) + " nor the per-head sizes fit the attention kernel's shared-memory tiles"; return 1; }
        } else if (type == "attention") {
            c.kind = MIX_WINDOW;
            c.G = (int)m.at("kv_heads").number(c.H);
            c.scale = (float)m.at("scale").number(1.0);
            c.window = m.has("mask") && m.at("mask").is_obj() ? (int)m.at("mask").at("size").number(0) : 0;
            if (c.window < 0) { error = where + ": mask.size must not be negative"; return 1; }
            if (!B::attention_fits(c.dk, c.dv)) { error = where + ": head dim " + std::to_string(c.dk) + " needs more shared memory than an SM has for the attention tiles"; return 1; }
        } else { error = where + ": unknown layer type '" + type + "'"; return 1; }
        if (c.H <= 0 || c.G <= 0 || c.dk <= 0 || c.dv <= 0 || c.H % c.G != 0) { error = where + ": bad head geometry"; return 1; }
        if (jl.has("mlp") && jl.at("mlp").is_obj()) {
            const Json& f = jl.at("mlp");
            const std::string kind = f.has("kind") ? f.at("kind").str : "moe";
            if (kind != "moe") { error = where + ": unknown mlp kind '" + kind + "'"; return 1; }
            c.moe.on = true;
            c.moe.ff = (int)f.at("expert").at("ff").number(0);
            const Json& r = f.at("router");
            c.moe.E = (int)r.at("experts").number(0); c.moe.top = (int)r.at("top").number(0);
            c.moe.scale = r.has("scale") ? (float)r.at("scale").number(1.0) : 1.0f;
            if (c.moe.ff <= 0 || c.moe.E <= 0 || c.moe.top <= 0 || c.moe.top > c.moe.E || c.moe.E > 4096) { error = where + ": bad expert geometry"; return 1; }
        }
        return 0;
    }

    // ---- weights -----------------------------------------------------------------------------------------------------------
    int load_norm(const SafeTensors& st, const std::string& name, int n, Norm& out) {
        const StTensor* t = nullptr;
        if (need(st, name, {n}, &t) || upload_f32(t, &out.w)) return 1;
        if (need(st, name + ".b", {n}, &t) || upload_f32(t, &out.b)) return 1;
        t = st.find(name + ".alpha");
        if (!t || t->numel() != 1 || (t->dtype != "BF16" && t->dtype != "F32")) { error = "tensor '" + name + ".alpha' must hold one number"; return 1; }
        return upload_f32(t, &out.alpha);
    }
    int load_vec(const SafeTensors& st, const std::string& name, int n, float** out) {
        const StTensor* t = nullptr;
        return need(st, name, {n}, &t) || upload_f32(t, out);
    }
    // matrices stacked into one: rows of `names` in order
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
    int load_vec_stack(const SafeTensors& st, const std::vector<std::pair<std::string, int>>& parts, int inner, float** out) {
        size_t total = 0;
        for (const auto& pr : parts) total += (size_t)pr.second * inner;
        std::vector<float> host;
        host.reserve(total);
        for (const auto& pr : parts) {
            const StTensor* t = nullptr;
            std::vector<int64_t> shape = {pr.second};
            if (inner > 1 || pr.first.find(".conv") != std::string::npos) shape.push_back(inner);
            if (need(st, pr.first, shape, &t)) return 1;
            for (size_t i = 0; i < t->numel(); i++)
                host.push_back(t->dtype == "BF16" ? bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(t->data)[i]) : reinterpret_cast<const float*>(t->data)[i]);
        }
        if (dalloc(out, host.size())) return 1;
        GCK(cudaMemcpy(*out, host.data(), host.size() * 4, cudaMemcpyHostToDevice));
        return 0;
    }
    int upload_host(const std::vector<float>& v, WT* dst) {
        if (std::is_same<WT, float>::value) { GCK(cudaMemcpy(dst, v.data(), v.size() * 4, cudaMemcpyHostToDevice)); return 0; }
        std::vector<__nv_bfloat16> tmp(v.size());
        for (size_t i = 0; i < v.size(); i++) tmp[i] = __float2bfloat16_rn(v[i]);
        GCK(cudaMemcpy(dst, tmp.data(), tmp.size() * 2, cudaMemcpyHostToDevice));
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
        if (load_norm(st, "final.norm", width, final_norm)) return 1;
        layers.resize(jl.arr.size());
        for (size_t li = 0; li < layers.size(); li++) {
            Layer& L = layers[li];
            if (parse_layer(jl.arr[li], li, L.c)) return 1;
            LayerCfg& c = L.c;
            const std::string p = "l" + std::to_string(li) + ".", q = p + "mix.";
            if (load_norm(st, p + "norm1", width, L.n1) || load_norm(st, p + "norm1b", width, L.n1b)) return 1;
            const int att_cols = c.H * c.dv;
            if (c.kind == MIX_WINDOW) {
                const int nq = c.H * c.dk, nk = c.G * c.dk, nv = c.G * c.dv;
                if (load_stack(st, {{q + "q", nq}, {q + "k", nk}, {q + "v", nv}}, width, &L.w_in, &L.in_rows)) return 1;
                if (load_vec_stack(st, {{q + "q.b", nq}, {q + "k.b", nk}, {q + "v.b", nv}}, 1, &L.b_in)) return 1;
                if (load_vec(st, q + "q.norm", nq, &L.qnorm) || load_vec(st, q + "k.norm", nk, &L.knorm) || load_vec(st, q + "r1", c.H, &L.r1) ||
                    load_vec(st, q + "r2", c.H, &L.r2))
                    return 1;
                if (dalloc(&L.kcache, (size_t)max_tokens * nk) || dalloc(&L.vcache, (size_t)max_tokens * nv)) return 1;
                max_qa = std::max(max_qa, nq);
                max_att = std::max(max_att, att_cols);
            } else if (c.kind == MIX_LATENT) {
                const int dq = c.dk + c.dr;
                if (load_stack(st, {{q + "dq", c.rq}, {q + "dkv", c.rk + c.dr}}, width, &L.w_in, &L.in_rows)) return 1;
                if (load_vec(st, q + "dq.norm", c.rq, &L.dq_norm) || load_vec(st, q + "dkv.norm", c.rk, &L.dkv_norm)) return 1;
                if (load_stack(st, {{q + "uq", c.H * dq}}, c.rq, &L.wuq, nullptr) || load_stack(st, {{q + "uv", c.H * c.dv}}, c.rk, &L.wuv, nullptr) ||
                    load_stack(st, {{q + "uk", c.H * c.dk}}, c.rk, &L.wuk, nullptr))
                    return 1;
                if (need(st, q + "uk", {c.H * c.dk, c.rk}, &t)) return 1;
                std::vector<float> tr((size_t)c.H * c.rk * c.dk);   // [h][r][d] <- uk[h*dn + d][r]
                for (int hh = 0; hh < c.H; hh++)
                    for (int d = 0; d < c.dk; d++)
                        for (int r = 0; r < c.rk; r++) {
                            const size_t src = ((size_t)hh * c.dk + d) * c.rk + r;
                            tr[((size_t)hh * c.rk + r) * c.dk + d] =
                                t->dtype == "BF16" ? bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(t->data)[src]) : reinterpret_cast<const float*>(t->data)[src];
                        }
                if (dalloc(&L.wukT, tr.size()) || upload_host(tr, L.wukT)) return 1;
                if (dalloc(&L.lcache, (size_t)max_tokens * (c.rk + c.dr)) || dalloc(&L.lcache_op, (size_t)max_tokens * c.rk)) return 1;
                max_kfull = std::max(max_kfull, c.H * dq); max_vfull = std::max(max_vfull, c.H * c.dv); max_knope = std::max(max_knope, c.H * c.dk);
                if (c.rot.dims > 0) {
                    std::vector<double> f;
                    double mult;
                    c.rot.freqs(f, mult);
                    if (this->angle_tables(c.rot.key(), f, mult, &L.rot_cos, &L.rot_sin)) return 1;
                }
                max_lat = std::max(max_lat, c.rq);
                max_qb = std::max(max_qb, c.H * dq);
                max_qn = std::max(max_qn, c.H * c.dk);
                max_qa = std::max(max_qa, c.H * (c.rk + c.dr));
                max_att = std::max(max_att, c.H * c.rk);
                max_att2 = std::max(max_att2, att_cols);
            } else {
                const int nqk = c.G * c.dk, nv = c.H * c.dv, C = 2 * nqk + nv;
                t = st.find(q + "a1");
                if (!t || t->shape.size() != 2) { error = "tensor '" + q + "a1' is missing"; return 1; }
                c.ra = (int)t->shape[0];
                t = st.find(q + "g1");
                if (!t || t->shape.size() != 2) { error = "tensor '" + q + "g1' is missing"; return 1; }
                c.rg = (int)t->shape[0];
                if (load_stack(st, {{q + "q", nqk}, {q + "k", nqk}, {q + "v", nv}, {q + "b", c.H}, {q + "a1", c.ra}, {q + "g1", c.rg}}, width, &L.w_in, &L.in_rows))
                    return 1;
                if (load_vec_stack(st, {{q + "q.conv", nqk}, {q + "k.conv", nqk}, {q + "v.conv", nv}}, c.taps, &L.wconv)) return 1;
                if (load_vec(st, q + "A_log", c.H, &L.a_log) || load_vec(st, q + "norm", c.dv, &L.onorm) || load_vec(st, q + "dt_bias", c.H * c.dk, &L.dt_bias))
                    return 1;
                if (load_stack(st, {{q + "a2", c.H * c.dk}}, c.ra, &L.wa2, nullptr) || load_stack(st, {{q + "g2", nv}}, c.rg, &L.wg2, nullptr)) return 1;
                if (dalloc(&L.state, (size_t)c.H * c.dk * c.dv) || dalloc(&L.tail, (size_t)std::max(c.taps - 1, 1) * C)) return 1;
                GCK(cudaMemset(L.state, 0, (size_t)c.H * c.dk * c.dv * 4));
                GCK(cudaMemset(L.tail, 0, (size_t)std::max(c.taps - 1, 1) * C * 4));
                has_state = true;
                max_qa = std::max(max_qa, C);
                max_lat = std::max(max_lat, c.ra + c.rg);
                max_fa = std::max(max_fa, c.H * c.dk);
                max_fb = std::max(max_fb, 2 * nv);
                max_att = std::max(max_att, att_cols);
            }
            if (load_stack(st, {{q + "o", width}}, att_cols, &L.wo, nullptr)) return 1;
            max_proj = std::max(max_proj, L.in_rows);
            max_H = std::max(max_H, c.H);
            max_dv = std::max(max_dv, c.kind == MIX_LATENT ? c.rk : c.dv);
            if (c.moe.on) {
                const MoeCfg& f = c.moe;
                if (load_norm(st, p + "norm2", width, L.n2) || load_norm(st, p + "norm2b", width, L.n2b)) return 1;
                if (load_vec_stack(st, {{p + "mlp.router", f.E}}, width, &L.router) || load_vec(st, p + "mlp.correction", f.E, &L.correction)) return 1;
                std::vector<std::pair<std::string, int>> gs, us, ds;
                for (int e = 0; e < f.E; e++) {
                    const std::string pe = p + "mlp.e" + std::to_string(e) + ".";
                    gs.push_back({pe + "gate", f.ff}); us.push_back({pe + "up", f.ff}); ds.push_back({pe + "down", width});
                }
                if (load_stack(st, gs, width, &L.wgate, nullptr) || load_stack(st, us, width, &L.wup, nullptr) || load_stack(st, ds, f.ff, &L.wdown, nullptr)) return 1;
                max_top = std::max(max_top, f.top); max_ff = std::max(max_ff, f.ff); max_E = std::max(max_E, f.E);
            }
        }
        if (dalloc(&d_tokens, (size_t)max_tokens) || dalloc(&d_logits, (size_t)vocab)) return 1;
        GCK(cudaMemset(d_tokens, 0, (size_t)max_tokens * 4));
        info.architecture = "Tudatar";
        info.model_type = 4;
        info.vocab = (uint32_t)vocab; info.width = (uint32_t)width; info.n_layers = (uint32_t)layers.size(); info.max_tokens = max_tokens;
        info.heads = (uint32_t)layers[0].c.H; info.kv_heads = (uint32_t)layers[0].c.G; info.head_dim = (uint32_t)layers[0].c.dk;
        info.ff = (uint32_t)layers[0].c.moe.ff; info.dtype = opt.dtype; info.eps = eps;
        return ensure_scratch(1);
    }

    int ensure_scratch(size_t rows) override {
        if (rows <= cap) return 0;
        drop_graphs();   // captured launches point into the old scratch
        for (void* p : {(void*)x, (void*)hn, (void*)d_rows, (void*)h, (void*)lat, (void*)qn, (void*)att, (void*)att2, (void*)xg, (void*)act, (void*)proj,
                        (void*)qa, (void*)qb, (void*)fa, (void*)fb, (void*)beta, (void*)part, (void*)y, (void*)wts, (void*)eidx, (void*)slot, (void*)row_of,
                        (void*)grp, (void*)rz})
            dfree(p);
        cap = 0;
        const size_t pairs = rows * std::max(max_top, 1);
        if (dalloc(&x, rows * width) || dalloc(&hn, rows * width) || dalloc(&d_rows, rows) || dalloc(&h, rows * width) ||
            dalloc(&lat, rows * std::max(max_lat, 1)) || dalloc(&qn, rows * std::max(max_qn, 1)) || dalloc(&att, rows * max_att) ||
            dalloc(&att2, rows * std::max(max_att2, 1)) || dalloc(&proj, rows * max_proj) || dalloc(&qa, rows * max_qa) ||
            dalloc(&qb, rows * std::max(max_qb, 1)) || dalloc(&fa, rows * std::max(max_fa, 1)) || dalloc(&fb, rows * std::max(max_fb, 1)) ||
            dalloc(&beta, rows * max_H) || dalloc(&part, (size_t)max_H * MAX_SPLIT * (max_dv + 2)) || dalloc(&xg, pairs * width) ||
            dalloc(&act, pairs * std::max(max_ff, 1)) || dalloc(&y, pairs * width) || dalloc(&wts, pairs) || dalloc(&eidx, pairs) ||
            dalloc(&slot, pairs) || dalloc(&row_of, pairs) || dalloc(&grp, (size_t)max_E + 1) || dalloc(&rz, rows * std::max(max_E, 1)))
            return 1;
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
    // the mixer's fused input projection of N1(x): proj = N1(x) . w_in^T (+ bias).  One row: the norm is the prologue of the
    // streaming kernel; many rows: h <- N1(x) first
    int in_proj(cudaStream_t st, const Layer& L, int T) {
        EpiParams<AT> e{}; e.out = proj; e.ldo = L.in_rows; e.scale = 1.0f; e.bias = L.b_in;
        if (T == 1) {
            GemvRowsParams<AT, WT> p{};
            p.x = x; p.tn = L.n1.view(); p.w = L.w_in; p.K = width; p.O = L.in_rows; p.e = e;
            return this->template launch_gemv<EPI_STORE, NORM_TANH>(st, p);
        }
        if (norm_rows(st, T, L.n1)) return 1;
        return this->template matmul<EPI_STORE>(st, T, h, width, L.w_in, nullptr, width, L.in_rows, e);
    }
    // h <- N(x) in the operand type
    int norm_rows(cudaStream_t st, int T, const Norm& n) {
        TanhNormRowsParams<AT> p{};
        p.x = x; p.ldx = width; p.n = n.view(); p.out = h; p.ldo = width; p.width = width;
        return launch_k("tanhnorm_rows_kernel", st, pdl_now, tanhnorm_rows_kernel<AT>, dim3(T), dim3(256), 0, p);
    }
    // x += N(att_in . wo^T)
    int out_proj(cudaStream_t st, int T, const AT* a, int K, const WT* wo, const Norm& n) {
        EpiParams<AT> e{};
        e.out = x; e.ldo = width; e.ls = n.w; e.lb = n.b; e.tanh_alpha = n.alpha;
        return this->template matmul<EPI_RESID>(st, T, a, K, wo, nullptr, K, width, e);
    }

    int mixer_window(cudaStream_t st, const Layer& L, int T, const PosSrc& ps, uint32_t pos_hint) {
        const LayerCfg& c = L.c;
        if (in_proj(st, L, T)) return 1;
        QkvJointNormParams np{};
        np.qkv = proj; np.ld = L.in_rows; np.H = c.H; np.G = c.G; np.dk = c.dk; np.dv = c.dv; np.wq = L.qnorm; np.wk = L.knorm; np.eps = info.eps;
        np.q_out = qa; np.kcache = L.kcache; np.vcache = L.vcache; np.ps = ps;
        if (launch_k("qkv_jointnorm_post_kernel", st, pdl_now, qkv_jointnorm_post_kernel<256>, dim3(T, 3), dim3(256), 0, np)) return 1;
        AttnRowsParams<AT> p{};
        p.q = qa; p.kcache = L.kcache; p.vcache = L.vcache; p.out = att;
        p.T = T; p.H = c.H; p.G = c.G; p.dk = c.dk; p.dv = c.dv; p.scale = c.scale; p.ps = ps;
        p.k_ld = c.G * c.dk; p.v_ld = c.G * c.dv; p.window = c.window; p.r1 = L.r1; p.r2 = L.r2;
        if (this->attention_launch(st, p, part, pos_hint)) return 1;
        return out_proj(st, T, att, c.H * c.dv, L.wo, L.n1b);
    }

    int mixer_latent(cudaStream_t st, const Layer& L, int T, const PosSrc& ps, uint32_t pos_hint) {
        const LayerCfg& c = L.c;
        const int dq = c.dk + c.dr, dl = c.rk + c.dr;
        if (in_proj(st, L, T)) return 1;
        LatentKvPostParams<AT> kp{};
        kp.in = proj; kp.ld = L.in_rows; kp.rq = c.rq; kp.rk = c.rk; kp.dr = c.dr; kp.wq = L.dq_norm; kp.wkv = L.dkv_norm; kp.eps = info.eps;
        kp.rot_dims = c.rot.dims; kp.rot_cos = L.rot_cos; kp.rot_sin = L.rot_sin; kp.cq_out = lat; kp.cache = L.lcache; kp.cache_op = L.lcache_op; kp.ps = ps;
        if (launch_k("latent_kv_post_kernel", st, pdl_now, latent_kv_post_kernel<AT>, dim3(T), dim3(256), 0, kp)) return 1;
        EpiParams<AT> eq{}; eq.out = qb; eq.ldo = c.H * dq; eq.scale = 1.0f;
        if (this->template matmul<EPI_STORE>(st, T, lat, c.rq, L.wuq, nullptr, c.rq, c.H * dq, eq)) return 1;
        LatentQPostParams<AT> qp{};
        qp.q = qb; qp.H = c.H; qp.dn = c.dk; qp.dr = c.dr; qp.rk = c.rk; qp.rot_dims = c.rot.dims; qp.rot_cos = L.rot_cos; qp.rot_sin = L.rot_sin;
        qp.qn_out = qn; qp.qabs = qa; qp.ps = ps;
        if (c.per_head_ok && (!c.latent_space_ok || (T >= latent_expand_rows && !ps.sp))) {
            // per-head form: keys and values of positions 0 .. n up-projected from the cached latents, then plain attention.
            // A graph-replayed step does not know its position on the host: it up-projects to the end of its 64-position
            // bucket (rows beyond the position are never read by the attention)
            int n = (int)ps.pos + T;
            if (ps.sp) n = (int)(pos_hint / ATT_KT + 1 < (uint32_t)MAX_SPLIT ? std::min<uint32_t>(max_tokens, (pos_hint / ATT_KT + 1) * ATT_KT) : max_tokens);
            if (!kfull && (dalloc(&kfull, (size_t)max_tokens * max_kfull) || dalloc(&vfull, (size_t)max_tokens * max_vfull) || dalloc(&knope, (size_t)max_tokens * max_knope)))
                return 1;
            qp.qfull = qa;
            if (launch_k("latent_q_post_kernel", st, pdl_now, latent_q_post_kernel<AT>, dim3(T, (c.H + 3) / 4), dim3(128), 0, qp)) return 1;
            EpiParams<AT> ek{}; ek.out = knope; ek.ldo = c.H * c.dk; ek.scale = 1.0f;
            if (this->template matmul<EPI_STORE>(st, n, L.lcache_op, c.rk, L.wuk, nullptr, c.rk, c.H * c.dk, ek)) return 1;
            EpiParams<AT> ev2{}; ev2.out = vfull; ev2.ldo = c.H * c.dv; ev2.scale = 1.0f;
            if (this->template matmul<EPI_STORE>(st, n, L.lcache_op, c.rk, L.wuv, nullptr, c.rk, c.H * c.dv, ev2)) return 1;
            LatentExpandParams xp{};
            xp.knope = knope; xp.cache = L.lcache; xp.kfull = kfull; xp.H = c.H; xp.dn = c.dk; xp.dr = c.dr; xp.rk = c.rk;
            if (launch_k("latent_expand_kernel", st, pdl_now, latent_expand_kernel, dim3(n), dim3(256), 0, xp)) return 1;
            AttnRowsParams<AT> p{};
            p.q = qa; p.kcache = kfull; p.vcache = vfull; p.out = att2;
            p.T = T; p.H = c.H; p.G = c.H; p.dk = dq; p.dv = c.dv; p.scale = c.scale; p.ps = ps; p.k_ld = c.H * dq; p.v_ld = c.H * c.dv;
            if (this->attention_launch(st, p, part, pos_hint)) return 1;
            return out_proj(st, T, att2, c.H * c.dv, L.wo, L.n1b);
        }
        if (launch_k("latent_q_post_kernel", st, pdl_now, latent_q_post_kernel<AT>, dim3(T, (c.H + 3) / 4), dim3(128), 0, qp)) return 1;
        // the unrotated query part of head z into the latent space: qa[:, z*dl .. z*dl+rk] = qn[:, z*dn ..] . wukT[z]^T
        EpiParams<AT> ea{}; ea.out = qa; ea.ldo = c.H * dl; ea.scale = 1.0f;
        if (this->template matmul_batched<EPI_STORE>(st, T, c.H, qn, c.H * c.dk, c.dk, L.wukT, (long long)c.rk * c.dk, c.dk, c.rk, ea, dl)) return 1;
        AttnRowsParams<AT> p{};   // one shared key/value head: keys [latent | rotated part], values = the latent
        p.q = qa; p.kcache = L.lcache; p.vcache = L.lcache; p.out = att;
        p.T = T; p.H = c.H; p.G = 1; p.dk = dl; p.dv = c.rk; p.scale = c.scale; p.ps = ps; p.k_ld = dl; p.v_ld = dl;
        if (this->attention_launch(st, p, part, pos_hint)) return 1;
        // values' up-projection per head: att2[:, z*dv ..] = att[:, z*rk ..] . wuv[z]^T
        EpiParams<AT> ev{}; ev.act = att2; ev.lda = c.H * c.dv;
        if (this->template matmul_batched<EPI_ACT>(st, T, c.H, att, c.H * c.rk, c.rk, L.wuv, (long long)c.dv * c.rk, c.rk, c.dv, ev, c.dv)) return 1;
        return out_proj(st, T, att2, c.H * c.dv, L.wo, L.n1b);
    }

    template <int NR, int LPC> int launch_scan(cudaStream_t st, const DeltaScanParams& sp) {
        constexpr int cols = DELTA_THREADS / LPC;
        const size_t smem = delta_scan_smem(NR, LPC);
        if (optin(delta_scan_kernel<NR, LPC>, smem)) return 1;
        return launch_k("delta_scan_kernel", st, pdl_now, delta_scan_kernel<NR, LPC>, dim3((sp.dv + cols - 1) / cols, sp.H), dim3(DELTA_THREADS), smem, sp);
    }
    int mixer_delta(cudaStream_t st, const Layer& L, int T, const PosSrc& ps) {
        const LayerCfg& c = L.c;
        const int nqk = c.G * c.dk, nv = c.H * c.dv, C = 2 * nqk + nv;
        if (in_proj(st, L, T)) return 1;
        AT* a_lat = lat;
        AT* g_lat = lat + (size_t)cap * c.ra;
        DeltaPreParams<AT> pp{};
        pp.in = proj; pp.ld = L.in_rows; pp.H = c.H; pp.G = c.G; pp.dk = c.dk; pp.dv = c.dv; pp.taps = c.taps; pp.ra = c.ra; pp.rg = c.rg;
        pp.wconv = L.wconv; pp.tail = L.tail; pp.qkv_out = qa; pp.beta = beta; pp.a_lat = a_lat; pp.g_lat = g_lat; pp.ps = ps;
        const int tasks = 2 * c.G + (nv + 127) / 128 + 1;
        if (launch_k("delta_pre_kernel", st, pdl_now, delta_pre_kernel<AT>, dim3(T, T >= 64 ? std::min(4, (tasks + 3) / 4) : std::min(16, (tasks + 3) / 4)), dim3(128), 0, pp))
            return 1;
        if (c.taps > 1) {
            ConvTailParams tp{};
            tp.in = proj; tp.ld = L.in_rows; tp.tail = L.tail; tp.C = C; tp.taps = c.taps; tp.T = T; tp.ps = ps;
            if (launch_k("conv_tail_update_kernel", st, pdl_now, conv_tail_update_kernel, dim3((C + 255) / 256), dim3(256), 0, tp)) return 1;
        }
        float* araw = fa;
        float* graw = fb;
        float* o = fb + (size_t)cap * nv;
        EpiParams<AT> ea{}; ea.out = araw; ea.ldo = c.H * c.dk; ea.scale = 1.0f; ea.bias = L.dt_bias;
        if (this->template matmul<EPI_STORE>(st, T, a_lat, c.ra, L.wa2, nullptr, c.ra, c.H * c.dk, ea)) return 1;
        EpiParams<AT> eg{}; eg.out = graw; eg.ldo = nv; eg.scale = 1.0f;
        if (this->template matmul<EPI_STORE>(st, T, g_lat, c.rg, L.wg2, nullptr, c.rg, nv, eg)) return 1;
        DeltaDecayParams dp{};
        dp.a = araw; dp.a_log = L.a_log; dp.n = T * c.H * c.dk; dp.H = c.H; dp.dk = c.dk;
        if (launch_k("delta_decay_kernel", st, pdl_now, delta_decay_kernel, dim3((dp.n + 255) / 256), dim3(256), 0, dp)) return 1;
        DeltaScanParams sp{};
        sp.qkv = qa; sp.ld = C; sp.decay = araw; sp.beta = beta; sp.state = L.state; sp.out = o;
        sp.T = T; sp.H = c.H; sp.G = c.G; sp.dk = c.dk; sp.dv = c.dv; sp.ps = ps;
        int nr, lpc;
        delta_scan_shape(c.dk, &nr, &lpc);
        int rc = 1;
        if (nr == 16 && lpc == 1) rc = launch_scan<16, 1>(st, sp);
        else if (nr == 16 && lpc == 2) rc = launch_scan<16, 2>(st, sp);
        else if (nr == 8 && lpc == 8) rc = launch_scan<8, 8>(st, sp);
        else if (nr == 8 && lpc == 16) rc = launch_scan<8, 16>(st, sp);
        else if (nr == 8 && lpc == 32) rc = launch_scan<8, 32>(st, sp);
        else rc = launch_scan<16, 32>(st, sp);
        if (rc) return 1;
        GatedHeadNormParams<AT> gp{};
        gp.o = o; gp.graw = graw; gp.w = L.onorm; gp.eps = info.eps; gp.out = att; gp.rows = T * c.H; gp.dv = c.dv;
        if (launch_k("gated_headnorm_kernel", st, pdl_now, gated_headnorm_kernel<AT>, dim3((gp.rows + 3) / 4), dim3(128), 0, gp)) return 1;
        return out_proj(st, T, att, nv, L.wo, L.n1b);
    }

    int experts(cudaStream_t st, const Layer& L, int T) {
        const MoeCfg& f = L.c.moe;
        // one row: the norm N2 is applied inside the kernels that read x (router logits, gate/up products); many rows: h <- N2(x)
        if (T > 1 && norm_rows(st, T, L.n2)) return 1;
        MoeRouterParams<AT> rp{};
        rp.h = T > 1 ? h : nullptr; rp.x = x; rp.tn = L.n2.view(); rp.ld = width; rp.router = L.router; rp.correction = L.correction;
        rp.E = f.E; rp.top = f.top; rp.width = width; rp.scale = f.scale; rp.z = rz; rp.idx = eidx; rp.wts = wts;
        if (launch_k("moe_logits_kernel", st, pdl_now, moe_logits_kernel<AT>, dim3(T, (f.E + 3) / 4), dim3(128), 0, rp)) return 1;
        if (launch_k("moe_topk_kernel", st, pdl_now, moe_topk_kernel<AT>, dim3(T), dim3(32), (size_t)2 * f.E * 4, rp)) return 1;
        MoeCombineParams cp{};
        cp.y = y; cp.wts = wts; cp.x = x; cp.ldx = width; cp.n = L.n2b.view(); cp.top = f.top; cp.width = width;
        EpiParams<AT> eg{}; eg.act = act; eg.lda = f.ff;
        EpiParams<AT> ed{}; ed.out = y; ed.ldo = width; ed.scale = 1.0f;
        if (T == 1) {   // the chosen experts' matrices, picked on the device from the router's list
            GemvRowsParams<AT, WT> p{};
            p.x = x; p.tn = L.n2.view(); p.w = L.wgate; p.w2 = L.wup; p.K = width; p.O = f.ff; p.e = eg; p.bidx = eidx;
            p.w_bs = (long long)f.ff * width; p.o_bs = f.ff;
            if (this->template launch_gemv<EPI_GLU, NORM_TANH>(st, p, f.top)) return 1;
            GemvRowsParams<AT, WT> d{};
            d.a = act; d.w = L.wdown; d.K = f.ff; d.O = width; d.e = ed; d.bidx = eidx; d.a_bs = f.ff; d.w_bs = (long long)width * f.ff; d.o_bs = width;
            if (this->template launch_gemv<EPI_STORE, NORM_NONE>(st, d, f.top)) return 1;
            cp.slot = nullptr;
        } else {
            const int n = T * f.top;
            MoeSortParams sp{};
            sp.idx = eidx; sp.n = n; sp.E = f.E; sp.top = f.top; sp.grp = grp; sp.slot = slot; sp.row_of = row_of;
            if (launch_k("moe_sort_kernel", st, pdl_now, moe_sort_kernel, dim3(1), dim3(1024), (size_t)2 * f.E * 4, sp)) return 1;
            MoeGatherParams<AT> gp{};
            gp.h = h; gp.ld = width; gp.row_of = row_of; gp.out = xg; gp.width = width;
            if (launch_k("moe_gather_kernel", st, pdl_now, moe_gather_kernel<AT>, dim3(n), dim3(128), 0, gp)) return 1;
            if (this->template matmul_grouped<EPI_GLU>(st, n, f.E, grp, T, xg, width, L.wgate, L.wup, width, f.ff, eg)) return 1;
            if (this->template matmul_grouped<EPI_STORE>(st, n, f.E, grp, T, act, f.ff, L.wdown, nullptr, f.ff, width, ed)) return 1;
            cp.slot = slot;
        }
        return launch_k("moe_combine_kernel", st, pdl_now, moe_combine_kernel, dim3(T, T >= 64 ? 1 : (width + 255) / 256), dim3(256), 0, cp);
    }

    int run_layers(cudaStream_t st, int T, const PosSrc& ps, uint32_t pos_hint) override {
        {
            EmbedRowsParams<WT> p{};
            p.embed = embed; p.bigram = nullptr; p.tokens = d_tokens; p.x = x; p.width = width; p.ps = ps;
            embed_rows_kernel<WT><<<T, 128, 0, st>>>(p);
            if (check_launch("embed_rows_kernel")) return 1;
        }
        for (size_t li = 0; li < layers.size(); li++) {
            const Layer& L = layers[li];
            int rc = L.c.kind == MIX_WINDOW ? mixer_window(st, L, T, ps, pos_hint) : (L.c.kind == MIX_LATENT ? mixer_latent(st, L, T, ps, pos_hint) : mixer_delta(st, L, T, ps));
            if (rc) return 1;
            if (L.c.moe.on) {
                if (experts(st, L, T)) return 1;
            }
            if (this->keep_layer(st, li, T)) return 1;
        }
        return 0;
    }
    int head_rows(cudaStream_t st, int m, const uint32_t* rows_dev, float* out) override {
        EpiParams<AT> e{}; e.out = out; e.ldo = vocab; e.scale = logit_scale;
        if (m == 1 && rows_dev == nullptr) {
            GemvRowsParams<AT, WT> p{};
            p.x = x; p.tn = final_norm.view(); p.w = head; p.K = width; p.O = vocab; p.e = e;
            return this->template launch_gemv<EPI_STORE, NORM_TANH>(st, p);
        }
        TanhNormRowsParams<AT> np{};
        np.x = x; np.ldx = width; np.rows = rows_dev; np.n = final_norm.view(); np.out = hn; np.ldo = width; np.width = width;
        if (launch_k("tanhnorm_rows_kernel", st, pdl_now, tanhnorm_rows_kernel<AT>, dim3(m), dim3(256), 0, np)) return 1;
        return this->template matmul<EPI_STORE>(st, m, hn, width, head, nullptr, width, vocab, e);
    }

    void set_model_option(const char* name, int value) override {
        if (!strcmp(name, "latent_expand_rows")) latent_expand_rows = std::max(2, value);
    }
    // test access: what a layer caches per position.  Windowed attention: K and V rows; latent attention: the latent and the
    // rotated key part (as "k" and "v"); delta-rule layers keep no per-position rows.
    int read_kv(cudaStream_t st, uint32_t layer, uint32_t pos0, uint32_t n, float* k_out, float* v_out) override {
        if (layer >= layers.size() || (size_t)pos0 + n > max_tokens) { error = "read_kv: out of range"; return 1; }
        const Layer& L = layers[layer];
        GCK(cudaStreamSynchronize(st));
        if (L.c.kind == MIX_WINDOW) {
            const size_t nk = (size_t)L.c.G * L.c.dk, nv = (size_t)L.c.G * L.c.dv;
            GCK(cudaMemcpy(k_out, L.kcache + pos0 * nk, n * nk * 4, cudaMemcpyDeviceToHost));
            GCK(cudaMemcpy(v_out, L.vcache + pos0 * nv, n * nv * 4, cudaMemcpyDeviceToHost));
        } else if (L.c.kind == MIX_LATENT) {
            const size_t dl = (size_t)L.c.rk + L.c.dr;
            GCK(cudaMemcpy2D(k_out, (size_t)L.c.rk * 4, L.lcache + pos0 * dl, dl * 4, (size_t)L.c.rk * 4, n, cudaMemcpyDeviceToHost));
            if (L.c.dr > 0) GCK(cudaMemcpy2D(v_out, (size_t)L.c.dr * 4, L.lcache + pos0 * dl + L.c.rk, dl * 4, (size_t)L.c.dr * 4, n, cudaMemcpyDeviceToHost));
        } else { error = "read_kv: a delta-rule layer keeps a state, not rows per position"; return 1; }
        return 0;
    }
};

ArchModel* tudatar_factory(const std::string& dir, const Json& cfg, const ArchOptions& opt, std::string& err) {
    ArchModel* m = nullptr;
    int rc;
    if (opt.dtype == ARCH_F32) {
        auto* g = new TudatarModel<float, float>();
        rc = g->load(dir, cfg, opt);
        m = g;
    } else {
        auto* g = new TudatarModel<__nv_bfloat16, __nv_bfloat16>();
        rc = g->load(dir, cfg, opt);
        m = g;
    }
    if (rc) { err = m->error; delete m; return nullptr; }
    return m;
}

}  // namespace

void register_tudatar() { arch_register("Tudatar", tudatar_factory); }

}  // namespace lmrs
