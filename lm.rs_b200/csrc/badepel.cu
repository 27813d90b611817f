// badepel.cu -- the Badepel architecture (arch.h): a decoder whose residual is SEVERAL streams per token.  Sublayer q of a
// layer (1: mixer, 2: feed-forward) reads a weighted sum of the streams through an RMS norm and writes its output back to every
// stream while the streams are mixed among themselves,
//     u = sum_s in_q[s] X[s];   y = sublayer(rms(u) w_q);   X'[t] = sum_s mix_q[s][t] X[s] + m out_q[t] y       (m = residual_mult)
// (a model without these tensors has one stream and the ordinary x <- x + m y).  Two kinds of sequence mixer, listed per layer
// in config.json "layers":
//   "parallel"  two mixers on the same input, left_scale * L + right_scale * R:
//               L  grouped-head attention: projections with biases, a short causal convolution over time on q, k and v, q and k
//                  RMS-normed over the whole projection with a weight, the first rot.dims dimensions of every head rotated in
//                  neighbouring pairs, scaled and soft-capped scores, a sliding window, and a softmax whose denominator holds one
//                  more entry of score 0 without a value
//               R  gated linear attention: S <- diag(a) S + k v^T, o = S^T q / sqrt(dim), with a decay per head and key channel
//                  a = sigmoid(W_a2 W_a1 h + b)^(1/tau); o RMS-normed per head with a weight and multiplied by silu(W_g h)
//   "delta"     gated delta rule: short causal convolution + SiLU on q, k, v, unit-length q and k, write strength
//               sigmoid(W_b h), one decay per head exp(-exp(A_log) softplus(W_a h + dt_bias)); output as for R
// and two kinds of feed-forward: "dense" (SiLU GLU) and "moe" (router logits with a bias, the `top` largest chosen, weights =
// softmax over the chosen logits; experts g = min(gate, limit), u = clamp(up, +-limit), W_down(g sigmoid(1.702 g)(u + 1)); an
// optional shared expert of the same form).  logits = head(rms(sum of the streams) w).  Everything model-specific comes from
// config.json and the tensor shapes; the kernels are the generic ones of dense_ops.cuh / mixer_ops.cuh / moe_ops.cuh /
// dense_gemm.cuh, the step / chunking / graph machinery is DenseModel's.  Caches are addressed by position like those of the
// other models; recurrent states and convolution tails continue from the previous step and restart when a step begins at
// position 0.
#include "dense_model.cuh"
#include "mixer_ops.cuh"
#include "moe_ops.cuh"

namespace lmrs {
namespace {

enum BdMixer { BD_PARALLEL = 0, BD_DELTA = 1 };
enum BdFf { BD_FF_NONE = 0, BD_FF_DENSE = 1, BD_FF_MOE = 2 };

struct BdLayerCfg {
    int kind = BD_PARALLEL;
    // attention (left of a parallel mixer), or the delta rule
    int H = 0, G = 0, dk = 0, dv = 0, taps = 0;
    float scale = 1.0f, softcap = 0.0f;
    int window = 0, rot_dims = 0;
    double rot_base = 10000.0;
    // gated linear attention (right of a parallel mixer)
    int rH = 0, rdk = 0, rdv = 0, ra = 0;
    float tau = 1.0f, left_scale = 1.0f, right_scale = 1.0f;
    // feed-forward
    int ff_kind = BD_FF_NONE;
    int ff = 0;
    float limit = INFINITY;
    int E = 0, top = 0;
    int shared_ff = 0;
    float shared_limit = INFINITY;
};

template <typename AT, typename WT> class BadepelModel : public DenseModel<AT, WT> {
  public:
    typedef DenseModel<AT, WT> B;
    using B::error; using B::launches; using B::info; using B::d_logits; using B::width; using B::vocab; using B::max_tokens;
    using B::sms; using B::d_tokens; using B::cap; using B::x; using B::hn; using B::d_rows; using B::MAX_SPLIT; using B::pdl_now;
    using B::dalloc; using B::dfree; using B::need; using B::upload_w; using B::upload_f32; using B::check_launch; using B::launch_k;
    using B::drop_graphs; using B::optin;

    struct Hc { const float *win = nullptr, *wout = nullptr, *mix = nullptr; };   // one sublayer's stream weights
    struct Layer {
        BdLayerCfg c;
        float *norm1 = nullptr, *norm2 = nullptr;
        Hc hc1, hc2;
        WT* w_in = nullptr; int in_rows = 0;   // fused input projection of the mixer
        float* b_in = nullptr;                  // its bias (parallel: zeros behind the attention's rows)
        WT* wo = nullptr; int wo_cols = 0;      // output projection (parallel: [left | right] side by side)
        float *wconv = nullptr, *tail = nullptr; int conv_ch = 0;
        // attention
        float *qnorm = nullptr, *knorm = nullptr, *sink = nullptr, *kcache = nullptr, *vcache = nullptr;
        const float *rot_cos = nullptr, *rot_sin = nullptr;
        // gated linear attention / delta rule
        WT* wa2 = nullptr;
        float *a2b = nullptr, *onorm = nullptr, *state = nullptr, *a_log = nullptr, *dt_bias = nullptr;
        // feed-forward
        WT *wgate = nullptr, *wup = nullptr, *wdown = nullptr;   // dense: [ff][width] x2, [width][ff]; moe: [E][ff][width] x2, [E][width][ff]
        float *router = nullptr, *router_b = nullptr;
        WT *sgate = nullptr, *sup = nullptr, *sdown = nullptr;   // shared expert
    };
    std::vector<Layer> layers;
    WT *embed = nullptr, *head = nullptr;
    float* final_norm = nullptr;
    float* ones = nullptr;       // [STREAMS_MAX]: the stream weights of a model without them
    int S = 1;                   // residual streams
    float mult = 1.0f;           // residual_mult
    uint32_t next_pos = 0;       // where the recurrent states and convolution tails stand
    // scratch for `cap` rows
    float *xs = nullptr, *proj = nullptr, *qa = nullptr, *fa = nullptr, *fo = nullptr, *beta = nullptr, *yf = nullptr, *part = nullptr,
          *rz = nullptr, *wts = nullptr, *ye = nullptr, *ysh = nullptr;
    AT *h = nullptr, *lat = nullptr, *att = nullptr, *act = nullptr, *xg = nullptr;
    int *eidx = nullptr, *slot = nullptr, *row_of = nullptr, *grp = nullptr;
    int max_proj = 0, max_ra = 0, max_qa = 0, max_fa = 0, max_fo = 0, max_H = 0, max_dv = 0, max_att = 0, max_act = 0, max_top = 0,
        max_eff = 0, max_E = 0;
    bool any_shared = false;
    int gla_lanes = 0;   // test / measurement override of the linear-attention scan's lanes per column at key sizes 33 .. 64

    size_t n_layers() const override { return layers.size(); }

    // ---- configuration ---------------------------------------------------------------------------------------------------
    int parse_layer(const Json& jl, size_t li, BdLayerCfg& c) {
        const std::string type = jl.at("type").str;
        const std::string where = "config.json layers[" + std::to_string(li) + "]";
        const Json& m = jl.at("mixer");
        if (type == "parallel") {
            c.kind = BD_PARALLEL;
            const Json& l = m.at("left");
            const Json& r = m.at("right");
            c.H = (int)l.at("heads").number(0); c.G = (int)l.at("kv_heads").number(c.H);
            c.dk = (int)l.at("dim").number(0); c.dv = (int)l.at("vdim").number(c.dk);
            c.taps = l.has("conv") ? (int)l.at("conv").number(0) : 0;
            c.scale = (float)l.at("scale").number(1.0);
            c.softcap = l.has("softcap") ? (float)l.at("softcap").number(0.0) : 0.0f;
            c.window = l.has("mask") && l.at("mask").is_obj() ? (int)l.at("mask").at("size").number(0) : 0;
            if (l.has("rot") && l.at("rot").is_obj()) {
                c.rot_dims = (int)l.at("rot").at("dims").number(0);
                c.rot_base = l.at("rot").at("base").number(10000.0);
            }
            c.rH = (int)r.at("heads").number(0); c.rdk = (int)r.at("dim").number(0); c.rdv = (int)r.at("vdim").number(c.rdk);
            c.tau = (float)r.at("tau").number(1.0);
            c.left_scale = m.has("left_scale") ? (float)m.at("left_scale").number(1.0) : 1.0f;
            c.right_scale = m.has("right_scale") ? (float)m.at("right_scale").number(1.0) : 1.0f;
            if (c.window < 0 || c.taps < 0 || c.taps > CONV_MAX_TAPS) { error = where + ": mask.size must not be negative and conv at most " + std::to_string(CONV_MAX_TAPS); return 1; }
            if (c.rot_dims < 0 || c.rot_dims > c.dk || c.rot_dims % 2 != 0) { error = where + ": rot.dims must be even and at most dim"; return 1; }
            if (c.rH <= 0 || c.rdk <= 0 || c.rdv <= 0 || c.rdk > DELTA_MAX_DK || c.tau <= 0.0f) { error = where + ": bad geometry of the right mixer"; return 1; }
            if (c.dk <= 0 || !B::attention_fits(c.dk, c.dv)) { error = where + ": head dim " + std::to_string(c.dk) + " / vdim " + std::to_string(c.dv) + " do not fit the attention kernel's shared-memory tiles"; return 1; }
        } else if (type == "delta") {
            c.kind = BD_DELTA;
            c.H = (int)m.at("heads").number(0); c.G = (int)m.at("kv_heads").number(c.H);
            c.dk = (int)m.at("dim").number(0); c.dv = (int)m.at("vdim").number(c.dk);
            c.taps = (int)m.at("conv").number(0);
            if (c.taps < 1 || c.taps > CONV_MAX_TAPS) { error = where + ": conv must be 1 .. " + std::to_string(CONV_MAX_TAPS); return 1; }
            if (c.dk > DELTA_MAX_DK) { error = where + ": dim above " + std::to_string(DELTA_MAX_DK) + " is not supported by the delta-rule kernel"; return 1; }
        } else { error = where + ": unknown layer type '" + type + "'"; return 1; }
        if (c.H <= 0 || c.G <= 0 || c.dk <= 0 || c.dv <= 0 || c.H % c.G != 0) { error = where + ": bad head geometry"; return 1; }
        if (jl.has("mlp") && jl.at("mlp").is_obj()) {
            const Json& f = jl.at("mlp");
            const std::string kind = f.has("kind") ? f.at("kind").str : "dense";
            if (kind == "dense") {
                c.ff_kind = BD_FF_DENSE;
                c.ff = (int)f.at("ff").number(0);
                if (c.ff <= 0) { error = where + ": mlp.ff is required"; return 1; }
            } else if (kind == "moe") {
                c.ff_kind = BD_FF_MOE;
                c.ff = (int)f.at("expert").at("ff").number(0);
                if (f.at("expert").has("limit")) c.limit = (float)f.at("expert").at("limit").number(INFINITY);
                c.E = (int)f.at("router").at("experts").number(0);
                c.top = (int)f.at("router").at("top").number(0);
                if (f.has("shared") && f.at("shared").is_obj()) {
                    c.shared_ff = (int)f.at("shared").at("ff").number(0);
                    if (f.at("shared").has("limit")) c.shared_limit = (float)f.at("shared").at("limit").number(INFINITY);
                }
                if (c.E <= 0 || c.ff <= 0 || c.top <= 0 || c.top > c.E || c.E > 4096 || c.shared_ff < 0) { error = where + ": bad expert geometry"; return 1; }
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
    // vectors ([n]) or tap tables ([n][inner]) laid end to end as f32, then `pad` zeros
    int load_f32_stack(const SafeTensors& st, const std::vector<std::pair<std::string, int>>& parts, int inner, int pad, float** out) {
        std::vector<float> host;
        for (const auto& pr : parts) {
            const StTensor* t = nullptr;
            std::vector<int64_t> shape = {pr.second};
            if (inner > 0) shape.push_back(inner);
            if (need(st, pr.first, shape, &t)) return 1;
            for (size_t i = 0; i < t->numel(); i++)
                host.push_back(t->dtype == "BF16" ? bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(t->data)[i]) : reinterpret_cast<const float*>(t->data)[i]);
        }
        host.resize(host.size() + (size_t)pad, 0.0f);
        if (dalloc(out, host.size())) return 1;
        GCK(cudaMemcpy(*out, host.data(), host.size() * 4, cudaMemcpyHostToDevice));
        return 0;
    }
    // two matrices with the same number of rows side by side: out [rows][K1 + K2]
    int load_side_by_side(const SafeTensors& st, const std::string& n1, int K1, const std::string& n2, int K2, int rows, WT** out) {
        if (dalloc(out, (size_t)rows * (K1 + K2))) return 1;
        const std::pair<std::string, int> parts[2] = {{n1, K1}, {n2, K2}};
        int c0 = 0;
        for (const auto& pr : parts) {
            const StTensor* t = nullptr;
            WT* tmp = nullptr;
            if (need(st, pr.first, {rows, pr.second}, &t)) return 1;
            GCK(cudaMalloc(&tmp, std::max<size_t>(t->numel(), 1) * sizeof(WT)));
            int rc = upload_w(t, tmp);
            cudaError_t e = cudaSuccess;
            if (!rc) e = cudaMemcpy2D(*out + c0, (size_t)(K1 + K2) * sizeof(WT), tmp, (size_t)pr.second * sizeof(WT), (size_t)pr.second * sizeof(WT), rows, cudaMemcpyDeviceToDevice);
            cudaFree(tmp);
            if (rc) return 1;
            GCK(e);
            c0 += pr.second;
        }
        return 0;
    }
    int load_hc(const SafeTensors& st, const std::string& name, Hc& out) {
        if (!st.find(name + ".in")) {
            if (S != 1) { error = "tensor '" + name + ".in' is missing (a model with several streams needs it)"; return 1; }
            out.win = out.wout = out.mix = ones;
            return 0;
        }
        float *a = nullptr, *b = nullptr, *m = nullptr;
        if (load_vec(st, name + ".in", S, &a) || load_vec(st, name + ".out", S, &b) || load_mat_f32(st, name + ".mix", S, S, &m)) return 1;
        out.win = a; out.wout = b; out.mix = m;
        return 0;
    }

    int load(const std::string& dir, const Json& cfg, const ArchOptions& opt) {
        sms = opt.sms;
        B::gemm_ctx.sms = opt.sms;
        width = (int)cfg.at("width").number(0);
        vocab = (int)cfg.at("vocab").number(0);
        if (width <= 0 || vocab <= 0) { error = "config.json: width and vocab are required"; return 1; }
        const float eps = (float)cfg.at("norm").at("eps").number(1e-6);
        S = cfg.has("streams") ? (int)cfg.at("streams").number(1) : 1;
        mult = cfg.has("residual_mult") ? (float)cfg.at("residual_mult").number(1.0) : 1.0f;
        if (S < 1 || S > STREAMS_MAX) { error = "config.json: streams must be 1 .. " + std::to_string(STREAMS_MAX); return 1; }
        max_tokens = opt.max_tokens ? opt.max_tokens : 4096u;
        const Json& jl = cfg.at("layers");
        if (jl.kind != Json::ARR || jl.arr.empty()) { error = "config.json: 'layers' must be a non-empty list"; return 1; }
        SafeTensors st;
        if (!st.open(dir + "/model.safetensors", error)) return 1;
        const StTensor* t = nullptr;
        if (need(st, "embed", {vocab, width}, &t) || dalloc(&embed, t->numel()) || upload_w(t, embed)) return 1;
        if (need(st, "head", {vocab, width}, &t) || dalloc(&head, t->numel()) || upload_w(t, head)) return 1;
        if (load_vec(st, "final.norm", width, &final_norm)) return 1;
        {
            std::vector<float> one(STREAMS_MAX, 1.0f);
            if (dalloc(&ones, one.size())) return 1;
            GCK(cudaMemcpy(ones, one.data(), one.size() * 4, cudaMemcpyHostToDevice));
        }
        layers.resize(jl.arr.size());
        for (size_t li = 0; li < layers.size(); li++) {
            Layer& L = layers[li];
            if (parse_layer(jl.arr[li], li, L.c)) return 1;
            BdLayerCfg& c = L.c;
            const std::string p = "l" + std::to_string(li) + ".", q = p + "mix.";
            if (load_vec(st, p + "norm1", width, &L.norm1) || load_hc(st, p + "hc1", L.hc1)) return 1;
            if (c.kind == BD_PARALLEL) {
                const std::string l = q + "left.", r = q + "right.";
                const int nq = c.H * c.dk, nk = c.G * c.dk, nv = c.G * c.dv, rqk = c.rH * c.rdk, rv = c.rH * c.rdv;
                t = st.find(r + "a1");
                if (!t || t->shape.size() != 2) { error = "tensor '" + r + "a1' is missing"; return 1; }
                c.ra = (int)t->shape[0];
                if (load_stack(st, {{l + "q", nq}, {l + "k", nk}, {l + "v", nv}, {r + "q", rqk}, {r + "k", rqk}, {r + "v", rv}, {r + "g", rv}, {r + "a1", c.ra}}, width,
                               &L.w_in, &L.in_rows))
                    return 1;
                if (load_f32_stack(st, {{l + "q.b", nq}, {l + "k.b", nk}, {l + "v.b", nv}}, 0, 2 * rqk + 2 * rv + c.ra, &L.b_in)) return 1;
                L.conv_ch = nq + nk + nv;
                if (c.taps > 0) {
                    if (load_f32_stack(st, {{l + "q.conv", nq}, {l + "k.conv", nk}, {l + "v.conv", nv}}, c.taps, 0, &L.wconv)) return 1;
                    if (dalloc(&L.tail, (size_t)std::max(c.taps - 1, 1) * L.conv_ch)) return 1;
                    GCK(cudaMemset(L.tail, 0, (size_t)std::max(c.taps - 1, 1) * L.conv_ch * 4));
                }
                if (load_vec(st, l + "q.norm", nq, &L.qnorm) || load_vec(st, l + "k.norm", nk, &L.knorm)) return 1;
                if (dalloc(&L.kcache, (size_t)max_tokens * nk) || dalloc(&L.vcache, (size_t)max_tokens * nv) || dalloc(&L.sink, (size_t)c.H)) return 1;
                GCK(cudaMemset(L.sink, 0, (size_t)c.H * 4));   // the extra softmax entry has score 0 for every head
                if (c.rot_dims > 0) {
                    std::vector<double> f;
                    for (int i = 0; i < c.rot_dims / 2; i++) f.push_back(pow(c.rot_base, -2.0 * (double)i / (double)c.rot_dims));
                    char key[160];
                    snprintf(key, sizeof key, "pairs/%d/%.17g", c.rot_dims, c.rot_base);
                    if (this->angle_tables(key, f, 1.0, &L.rot_cos, &L.rot_sin)) return 1;
                }
                if (load_stack(st, {{r + "a2", rqk}}, c.ra, &L.wa2, nullptr) ||
                    load_vec(st, r + "a2.b", rqk, &L.a2b) || load_vec(st, r + "norm", c.rdv, &L.onorm))
                    return 1;
                if (dalloc(&L.state, (size_t)c.rH * c.rdk * c.rdv)) return 1;
                GCK(cudaMemset(L.state, 0, (size_t)c.rH * c.rdk * c.rdv * 4));
                L.wo_cols = c.H * c.dv + rv;
                if (load_side_by_side(st, l + "o", c.H * c.dv, r + "o", rv, width, &L.wo)) return 1;
                max_ra = std::max(max_ra, c.ra);
                max_qa = std::max(max_qa, nq);
                max_fa = std::max(max_fa, rqk);
                max_fo = std::max(max_fo, rv);
                max_H = std::max(max_H, c.H);
                max_dv = std::max(max_dv, c.dv);
            } else {
                const int nqk = c.G * c.dk, nv = c.H * c.dv;
                L.conv_ch = 2 * nqk + nv;
                if (load_stack(st, {{q + "q", nqk}, {q + "k", nqk}, {q + "v", nv}, {q + "b", c.H}, {q + "a", c.H}, {q + "g", nv}}, width, &L.w_in, &L.in_rows)) return 1;
                if (load_f32_stack(st, {{q + "q.conv", nqk}, {q + "k.conv", nqk}, {q + "v.conv", nv}}, c.taps, 0, &L.wconv)) return 1;
                if (load_vec(st, q + "A_log", c.H, &L.a_log) || load_vec(st, q + "dt_bias", c.H, &L.dt_bias) || load_vec(st, q + "norm", c.dv, &L.onorm)) return 1;
                if (dalloc(&L.state, (size_t)c.H * c.dk * c.dv) || dalloc(&L.tail, (size_t)std::max(c.taps - 1, 1) * L.conv_ch)) return 1;
                GCK(cudaMemset(L.state, 0, (size_t)c.H * c.dk * c.dv * 4));
                GCK(cudaMemset(L.tail, 0, (size_t)std::max(c.taps - 1, 1) * L.conv_ch * 4));
                L.wo_cols = nv;
                if (load_stack(st, {{q + "o", width}}, nv, &L.wo, nullptr)) return 1;
                max_qa = std::max(max_qa, L.conv_ch);
                max_fa = std::max(max_fa, c.H);
                max_fo = std::max(max_fo, nv);
                max_H = std::max(max_H, c.H);
            }
            max_proj = std::max(max_proj, L.in_rows);
            max_att = std::max(max_att, L.wo_cols);
            if (c.ff_kind != BD_FF_NONE && (load_vec(st, p + "norm2", width, &L.norm2) || load_hc(st, p + "hc2", L.hc2))) return 1;
            if (c.ff_kind == BD_FF_DENSE) {
                if (load_stack(st, {{p + "mlp.gate", c.ff}}, width, &L.wgate, nullptr) || load_stack(st, {{p + "mlp.up", c.ff}}, width, &L.wup, nullptr) ||
                    load_stack(st, {{p + "mlp.down", width}}, c.ff, &L.wdown, nullptr))
                    return 1;
                max_act = std::max(max_act, c.ff);
            } else if (c.ff_kind == BD_FF_MOE) {
                if (load_mat_f32(st, p + "mlp.router", c.E, width, &L.router)) return 1;
                if (st.find(p + "mlp.router.b") && load_vec(st, p + "mlp.router.b", c.E, &L.router_b)) return 1;
                std::vector<std::pair<std::string, int>> gs, us, ds;
                for (int e = 0; e < c.E; e++) {
                    const std::string pe = p + "mlp.e" + std::to_string(e) + ".";
                    gs.push_back({pe + "gate", c.ff}); us.push_back({pe + "up", c.ff}); ds.push_back({pe + "down", width});
                }
                if (load_stack(st, gs, width, &L.wgate, nullptr) || load_stack(st, us, width, &L.wup, nullptr) || load_stack(st, ds, c.ff, &L.wdown, nullptr)) return 1;
                if (c.shared_ff > 0) {
                    if (load_stack(st, {{p + "mlp.shared.gate", c.shared_ff}}, width, &L.sgate, nullptr) ||
                        load_stack(st, {{p + "mlp.shared.up", c.shared_ff}}, width, &L.sup, nullptr) ||
                        load_stack(st, {{p + "mlp.shared.down", width}}, c.shared_ff, &L.sdown, nullptr))
                        return 1;
                    any_shared = true;
                    max_act = std::max(max_act, c.shared_ff);
                }
                max_top = std::max(max_top, c.top); max_eff = std::max(max_eff, c.ff); max_E = std::max(max_E, c.E);
            }
        }
        if (dalloc(&d_tokens, (size_t)max_tokens) || dalloc(&d_logits, (size_t)vocab)) return 1;
        GCK(cudaMemset(d_tokens, 0, (size_t)max_tokens * 4));
        info.architecture = "Badepel";
        info.model_type = 6;
        info.vocab = (uint32_t)vocab; info.width = (uint32_t)width; info.n_layers = (uint32_t)layers.size(); info.max_tokens = max_tokens;
        info.heads = (uint32_t)layers[0].c.H; info.kv_heads = (uint32_t)layers[0].c.G; info.head_dim = (uint32_t)layers[0].c.dk;
        info.ff = (uint32_t)layers[0].c.ff; info.dtype = opt.dtype; info.eps = eps;
        return ensure_scratch(1);
    }

    int ensure_scratch(size_t rows) override {
        if (rows <= cap) return 0;
        drop_graphs();   // captured launches point into the old scratch
        for (void* p : {(void*)x, (void*)hn, (void*)d_rows, (void*)xs, (void*)h, (void*)lat, (void*)att, (void*)act, (void*)xg, (void*)proj, (void*)qa,
                        (void*)fa, (void*)fo, (void*)beta, (void*)yf, (void*)part, (void*)rz, (void*)wts, (void*)ye, (void*)ysh, (void*)eidx, (void*)slot,
                        (void*)row_of, (void*)grp})
            dfree(p);
        x = nullptr; hn = nullptr; d_rows = nullptr; xs = nullptr; h = nullptr; lat = nullptr; att = nullptr; act = nullptr; xg = nullptr; proj = nullptr;
        qa = nullptr; fa = nullptr; fo = nullptr; beta = nullptr; yf = nullptr; part = nullptr; rz = nullptr; wts = nullptr; ye = nullptr; ysh = nullptr;
        eidx = nullptr; slot = nullptr; row_of = nullptr; grp = nullptr;
        cap = 0;
        const size_t pairs = rows * std::max(max_top, 1);
        const size_t act_n = std::max(rows * (size_t)std::max(max_act, 1), pairs * (size_t)std::max(max_eff, 1));
        if (dalloc(&x, rows * width) || dalloc(&hn, rows * width) || dalloc(&d_rows, rows) || dalloc(&xs, rows * S * width) || dalloc(&h, rows * width) ||
            dalloc(&lat, rows * std::max(max_ra, 1)) || dalloc(&att, rows * max_att) || dalloc(&act, act_n) || dalloc(&proj, rows * max_proj) ||
            dalloc(&qa, rows * std::max(max_qa, 1)) || dalloc(&fa, rows * std::max(max_fa, 1)) || dalloc(&fo, rows * std::max(max_fo, 1)) ||
            dalloc(&beta, rows * std::max(max_H, 1)) || dalloc(&yf, rows * width) || dalloc(&part, (size_t)std::max(max_H, 1) * MAX_SPLIT * (max_dv + 2)))
            return 1;
        if (max_top > 0 &&
            (dalloc(&xg, pairs * width) || dalloc(&rz, rows * max_E) || dalloc(&wts, pairs) || dalloc(&ye, pairs * width) || dalloc(&eidx, pairs) ||
             dalloc(&slot, pairs) || dalloc(&row_of, pairs) || dalloc(&grp, (size_t)max_E + 1)))
            return 1;
        if (any_shared && dalloc(&ysh, rows * width)) return 1;
        cap = rows;
        return 0;
    }

    // every mixer carries state that is not addressed by position (recurrent matrices, convolution tails): a step continues
    // where the last one ended or starts a new sequence at 0
    int begin_step(uint32_t pos, size_t n) override {
        if (pos != 0 && pos != next_pos) {
            error = "a model with recurrent layers continues at position " + std::to_string(next_pos) + " or restarts at 0, not at " + std::to_string(pos);
            return 1;
        }
        next_pos = pos + (uint32_t)n;
        return 0;
    }

    // ---- the residual streams ---------------------------------------------------------------------------------------------------
    struct Pending { const float* y = nullptr; const Hc* hc = nullptr; };   // a sublayer output that the streams have not taken in yet
    // one pass over the streams of T tokens: start them from the embedding rows (init), take in the pending sublayer output, and
    // read for the next sublayer (rd, through the norm nw into h) or sum the streams into x (sum_to_x)
    int streams_step(cudaStream_t st, int T, bool init, Pending& pend, const Hc* rd, const float* nw, bool sum_to_x) {
        StreamsParams<AT> p{};
        p.xs = xs; p.S = S; p.width = width;
        if (init) { p.init = x; p.ld_init = width; }
        if (pend.y) { p.y = pend.y; p.ldy = width; p.mix = pend.hc->mix; p.wout = pend.hc->wout; p.mult = mult; }
        if (rd) { p.win = rd->win; p.nw = nw; p.eps = info.eps; p.h = h; p.ldh = width; }
        if (sum_to_x) { p.sum_all = 1; p.u_out = x; p.ldu = width; }
        pend = Pending{};
        // a few tokens: one column or two per thread, so that the row's loads are all in flight at once
        const dim3 grid(T), block(T <= 8 && width > 512 ? 1024 : 256);
        if (S <= 1) return launch_k("streams_step_kernel", st, pdl_now, streams_step_kernel<AT, 1>, grid, block, 0, p);
        if (S <= 2) return launch_k("streams_step_kernel", st, pdl_now, streams_step_kernel<AT, 2>, grid, block, 0, p);
        if (S <= 4) return launch_k("streams_step_kernel", st, pdl_now, streams_step_kernel<AT, 4>, grid, block, 0, p);
        if (S <= 8) return launch_k("streams_step_kernel", st, pdl_now, streams_step_kernel<AT, 8>, grid, block, 0, p);
        return launch_k("streams_step_kernel", st, pdl_now, streams_step_kernel<AT, STREAMS_MAX>, grid, block, 0, p);
    }

    // ---- the layers -----------------------------------------------------------------------------------------------------------
    int in_proj(cudaStream_t st, const Layer& L, int T) {
        EpiParams<AT> e{}; e.out = proj; e.ldo = L.in_rows; e.scale = 1.0f; e.bias = L.b_in;
        return this->template matmul<EPI_STORE>(st, T, h, width, L.w_in, nullptr, width, L.in_rows, e);
    }
    int out_proj(cudaStream_t st, int T, const AT* a, int K, const WT* wo) {
        EpiParams<AT> e{}; e.out = yf; e.ldo = width; e.scale = 1.0f;
        return this->template matmul<EPI_STORE>(st, T, a, K, wo, nullptr, K, width, e);
    }
    int tail_update(cudaStream_t st, const Layer& L, int T, const PosSrc& ps) {
        if (L.c.taps <= 1) return 0;
        ConvTailParams tp{};
        tp.in = proj; tp.ld = L.in_rows; tp.tail = L.tail; tp.C = L.conv_ch; tp.taps = L.c.taps; tp.T = T; tp.ps = ps;
        return launch_k("conv_tail_update_kernel", st, pdl_now, conv_tail_update_kernel, dim3((L.conv_ch + 255) / 256), dim3(256), 0, tp);
    }
    template <int NR, int LPC, int MODE> int launch_scan(cudaStream_t st, const DeltaScanParams& sp) {
        constexpr int cols = DELTA_THREADS / LPC;
        const size_t smem = delta_scan_smem(NR, LPC);
        if (optin(delta_scan_kernel<NR, LPC, MODE>, smem)) return 1;
        return launch_k("delta_scan_kernel", st, pdl_now, delta_scan_kernel<NR, LPC, MODE>, dim3((sp.dv + cols - 1) / cols, sp.H), dim3(DELTA_THREADS), smem, sp);
    }
    template <int MODE> int scan(cudaStream_t st, const DeltaScanParams& sp) {
        int nr, lpc;
        delta_scan_shape(sp.dk, &nr, &lpc);
        if (MODE == SCAN_PLAIN && sp.dk > 32 && sp.dk <= 64) {   // no reduction sits on the way to the next token's state here
            const int lanes = gla_lanes > 0 ? gla_lanes : 8;
            if (lanes == 4) return launch_scan<16, 4, SCAN_PLAIN>(st, sp);
            if (lanes == 16) return launch_scan<4, 16, SCAN_PLAIN>(st, sp);
        }
        if (nr == 16 && lpc == 1) return launch_scan<16, 1, MODE>(st, sp);
        if (nr == 16 && lpc == 2) return launch_scan<16, 2, MODE>(st, sp);
        if (nr == 8 && lpc == 8) return launch_scan<8, 8, MODE>(st, sp);
        if (nr == 8 && lpc == 16) return launch_scan<8, 16, MODE>(st, sp);
        if (nr == 8 && lpc == 32) return launch_scan<8, 32, MODE>(st, sp);
        return launch_scan<16, 32, MODE>(st, sp);
    }
    // o / rms(o) * w * silu(gate logits of proj from column g_off) * out_scale -> att columns out_off ..
    int gated_norm(cudaStream_t st, const Layer& L, int T, int H, int dv, int g_off, int out_off, float out_scale) {
        GatedHeadNormParams<AT> gp{};
        gp.o = fo; gp.graw = proj + g_off; gp.w = L.onorm; gp.eps = info.eps; gp.out = att + out_off; gp.rows = T * H; gp.dv = dv;
        gp.gate_silu = 1; gp.H = H; gp.g_ld = L.in_rows; gp.out_ld = L.wo_cols; gp.has_out_scale = 1; gp.out_scale = out_scale;
        return launch_k("gated_headnorm_kernel", st, pdl_now, gated_headnorm_kernel<AT>, dim3((gp.rows + 3) / 4), dim3(128), 0, gp);
    }

    int mixer_parallel(cudaStream_t st, const Layer& L, int T, const PosSrc& ps, uint32_t pos_hint) {
        const BdLayerCfg& c = L.c;
        const int nq = c.H * c.dk, nk = c.G * c.dk, nv = c.G * c.dv, rqk = c.rH * c.rdk, rv = c.rH * c.rdv;
        const int r_off = nq + nk + nv, kl = c.H * c.dv;
        if (in_proj(st, L, T)) return 1;
        {   // the decay's low-rank row (the last columns of the projection) in the operand type, for the second half of that projection
            CastColsParams<AT> cp{};
            cp.in = proj + r_off + 2 * rqk + 2 * rv; cp.ld = L.in_rows; cp.out = lat; cp.ldo = c.ra; cp.n = c.ra; cp.total = T * c.ra;
            if (launch_k("cast_cols_kernel", st, pdl_now, cast_cols_kernel<AT>, dim3((cp.total + 255) / 256), dim3(256), 0, cp)) return 1;
        }
        // left: convolution, whole-row norms, rotation, cache rows; then the window attention into the left columns
        QkvJointNormParams np{};
        np.qkv = proj; np.ld = L.in_rows; np.H = c.H; np.G = c.G; np.dk = c.dk; np.dv = c.dv; np.wq = L.qnorm; np.wk = L.knorm; np.eps = info.eps;
        np.q_out = qa; np.kcache = L.kcache; np.vcache = L.vcache; np.ps = ps; np.taps = c.taps; np.wconv = L.wconv; np.tail = L.tail;
        np.rot_dims = c.rot_dims; np.rot_cos = L.rot_cos; np.rot_sin = L.rot_sin; np.v_plain = 1;
        const size_t jn_smem = c.taps > 0 ? (size_t)std::max(nq, nk) * 4 : 0;
        if (T == 1 && c.taps > 1) np.tail_out = L.tail;   // one token: the kernel moves the tail on itself
        if (T <= 8) {
            if (optin(qkv_jointnorm_post_kernel<1024>, jn_smem)) return 1;
            if (launch_k("qkv_jointnorm_post_kernel", st, pdl_now, qkv_jointnorm_post_kernel<1024>, dim3(T, 3), dim3(1024), jn_smem, np)) return 1;
        } else {
            if (optin(qkv_jointnorm_post_kernel<256>, jn_smem)) return 1;
            if (launch_k("qkv_jointnorm_post_kernel", st, pdl_now, qkv_jointnorm_post_kernel<256>, dim3(T, 3), dim3(256), jn_smem, np)) return 1;
        }
        if (!np.tail_out && tail_update(st, L, T, ps)) return 1;
        AttnRowsParams<AT> p{};
        p.q = qa; p.kcache = L.kcache; p.vcache = L.vcache; p.out = att;
        p.T = T; p.H = c.H; p.G = c.G; p.dk = c.dk; p.dv = c.dv; p.scale = c.scale; p.softcap = c.softcap; p.ps = ps;
        p.k_ld = nk; p.v_ld = nv; p.window = c.window; p.sink = L.sink; p.out_ld = L.wo_cols; p.has_out_scale = 1; p.out_scale = c.left_scale;
        if (this->attention_launch(st, p, part, pos_hint)) return 1;
        // right: decays, the recurrence, head norm and gate into the right columns
        EpiParams<AT> ea{}; ea.out = fa; ea.ldo = rqk; ea.scale = 1.0f; ea.bias = L.a2b;
        if (this->template matmul<EPI_STORE>(st, T, lat, c.ra, L.wa2, nullptr, c.ra, rqk, ea)) return 1;
        DeltaDecayParams dp{};
        dp.a = fa; dp.a_log = nullptr; dp.n = T * rqk; dp.H = c.rH; dp.dk = c.rdk; dp.inv_tau = 1.0f / c.tau;
        if (launch_k("delta_decay_kernel", st, pdl_now, delta_decay_kernel, dim3((dp.n + 255) / 256), dim3(256), 0, dp)) return 1;
        DeltaScanParams sp{};
        sp.qkv = proj + r_off; sp.ld = L.in_rows; sp.decay = fa; sp.beta = nullptr; sp.state = L.state; sp.out = fo;
        sp.T = T; sp.H = c.rH; sp.G = c.rH; sp.dk = c.rdk; sp.dv = c.rdv; sp.ps = ps; sp.q_scale = 1.0f / sqrtf((float)c.rdk);
        if (scan<SCAN_PLAIN>(st, sp)) return 1;
        if (gated_norm(st, L, T, c.rH, c.rdv, r_off + 2 * rqk + rv, kl, c.right_scale)) return 1;
        return out_proj(st, T, att, L.wo_cols, L.wo);
    }

    int mixer_delta(cudaStream_t st, const Layer& L, int T, const PosSrc& ps) {
        const BdLayerCfg& c = L.c;
        const int nqk = c.G * c.dk, nv = c.H * c.dv, C = L.conv_ch;
        if (in_proj(st, L, T)) return 1;
        DeltaPreParams<AT> pp{};
        pp.in = proj; pp.ld = L.in_rows; pp.H = c.H; pp.G = c.G; pp.dk = c.dk; pp.dv = c.dv; pp.taps = c.taps; pp.ra = 0; pp.rg = 0;
        pp.wconv = L.wconv; pp.tail = L.tail; pp.qkv_out = qa; pp.beta = beta; pp.ps = ps;
        pp.head_decay = fa; pp.a_log = L.a_log; pp.dt_bias = L.dt_bias;
        const int tasks = 2 * c.G + (nv + 127) / 128 + 1;
        if (launch_k("delta_pre_kernel", st, pdl_now, delta_pre_kernel<AT>, dim3(T, T >= 64 ? std::min(4, (tasks + 3) / 4) : std::min(16, (tasks + 3) / 4)), dim3(128), 0, pp))
            return 1;
        if (tail_update(st, L, T, ps)) return 1;
        DeltaScanParams sp{};
        sp.qkv = qa; sp.ld = C; sp.decay = fa; sp.beta = beta; sp.state = L.state; sp.out = fo;
        sp.T = T; sp.H = c.H; sp.G = c.G; sp.dk = c.dk; sp.dv = c.dv; sp.ps = ps;
        if (scan<SCAN_DELTA_HEAD>(st, sp)) return 1;
        if (gated_norm(st, L, T, c.H, c.dv, C + 2 * c.H, 0, 1.0f)) return 1;
        (void)nqk;
        return out_proj(st, T, att, nv, L.wo);
    }

    int ff_dense(cudaStream_t st, const Layer& L, int T) {
        const BdLayerCfg& c = L.c;
        EpiParams<AT> eg{}; eg.act = act; eg.lda = c.ff; eg.glu_kind = GLU_SILU;
        if (this->template matmul<EPI_GLU>(st, T, h, width, L.wgate, L.wup, width, c.ff, eg)) return 1;
        return out_proj(st, T, act, c.ff, L.wdown);
    }

    int ff_moe(cudaStream_t st, const Layer& L, int T) {
        const BdLayerCfg& c = L.c;
        MoeRouterParams<AT> rp{};
        rp.h = h; rp.ld = width; rp.router = L.router; rp.bias = L.router_b; rp.E = c.E; rp.top = c.top; rp.width = width; rp.softmax = 2;
        rp.scale = 1.0f; rp.z = rz; rp.idx = eidx; rp.wts = wts;
        if (launch_k("moe_logits_kernel", st, pdl_now, moe_logits_kernel<AT>, dim3(T, (c.E + 3) / 4), dim3(128), 0, rp)) return 1;
        if (launch_k("moe_topk_kernel", st, pdl_now, moe_topk_kernel<AT>, dim3(T), dim3(32), (size_t)2 * c.E * 4, rp)) return 1;
        MoeCombineParams cp{};
        cp.y = ye; cp.wts = wts; cp.top = c.top; cp.width = width; cp.out = yf; cp.ldo = width;
        EpiParams<AT> eg{}; eg.act = act; eg.lda = c.ff; eg.glu_kind = GLU_CLAMPED; eg.glu_limit = c.limit; eg.glu_alpha = 1.702f;
        EpiParams<AT> ed{}; ed.out = ye; ed.ldo = width; ed.scale = 1.0f;
        if (T == 1) {   // the chosen experts' matrices, picked on the device from the router's list
            GemvRowsParams<AT, WT> u{};
            u.a = h; u.w = L.wgate; u.w2 = L.wup; u.K = width; u.O = c.ff; u.e = eg; u.bidx = eidx; u.w_bs = (long long)c.ff * width; u.o_bs = c.ff;
            if (this->template launch_gemv<EPI_GLU, NORM_NONE>(st, u, c.top)) return 1;
            GemvRowsParams<AT, WT> d{};
            d.a = act; d.w = L.wdown; d.K = c.ff; d.O = width; d.e = ed; d.bidx = eidx; d.a_bs = c.ff; d.w_bs = (long long)width * c.ff; d.o_bs = width;
            if (this->template launch_gemv<EPI_STORE, NORM_NONE>(st, d, c.top)) return 1;
            cp.slot = nullptr;
        } else {   // rows sorted by expert
            const int n = T * c.top;
            MoeSortParams sp{};
            sp.idx = eidx; sp.n = n; sp.E = c.E; sp.top = c.top; sp.grp = grp; sp.slot = slot; sp.row_of = row_of;
            if (launch_k("moe_sort_kernel", st, pdl_now, moe_sort_kernel, dim3(1), dim3(1024), (size_t)2 * c.E * 4, sp)) return 1;
            MoeGatherParams<AT> gp{};
            gp.h = h; gp.ld = width; gp.row_of = row_of; gp.out = xg; gp.width = width;
            if (launch_k("moe_gather_kernel", st, pdl_now, moe_gather_kernel<AT>, dim3(n), dim3(128), 0, gp)) return 1;
            if (this->template matmul_grouped<EPI_GLU>(st, n, c.E, grp, T, xg, width, L.wgate, L.wup, width, c.ff, eg)) return 1;
            if (this->template matmul_grouped<EPI_STORE>(st, n, c.E, grp, T, act, c.ff, L.wdown, nullptr, c.ff, width, ed)) return 1;
            cp.slot = slot;
        }
        if (c.shared_ff > 0) {
            EpiParams<AT> sg{}; sg.act = act; sg.lda = c.shared_ff; sg.glu_kind = GLU_CLAMPED; sg.glu_limit = c.shared_limit; sg.glu_alpha = 1.702f;
            if (this->template matmul<EPI_GLU>(st, T, h, width, L.sgate, L.sup, width, c.shared_ff, sg)) return 1;
            EpiParams<AT> sd{}; sd.out = ysh; sd.ldo = width; sd.scale = 1.0f;
            if (this->template matmul<EPI_STORE>(st, T, act, c.shared_ff, L.sdown, nullptr, c.shared_ff, width, sd)) return 1;
            cp.add = ysh;
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
        Pending pend;
        for (size_t li = 0; li < layers.size(); li++) {
            const Layer& L = layers[li];
            if (streams_step(st, T, li == 0, pend, &L.hc1, L.norm1, false)) return 1;
            if (L.c.kind == BD_PARALLEL ? mixer_parallel(st, L, T, ps, pos_hint) : mixer_delta(st, L, T, ps)) return 1;
            pend.y = yf; pend.hc = &L.hc1;
            if (L.c.ff_kind != BD_FF_NONE) {
                if (streams_step(st, T, false, pend, &L.hc2, L.norm2, false)) return 1;
                if (L.c.ff_kind == BD_FF_DENSE ? ff_dense(st, L, T) : ff_moe(st, L, T)) return 1;
                pend.y = yf; pend.hc = &L.hc2;
            }
            if (B::keep_layers || li + 1 == layers.size()) {   // the sum of the streams: a layer's output for a test, the final norm's input
                if (streams_step(st, T, false, pend, nullptr, nullptr, true)) return 1;
                if (this->keep_layer(st, li, T)) return 1;
            }
        }
        return 0;
    }
    int head_rows(cudaStream_t st, int m, const uint32_t* rows_dev, float* out) override {
        EpiParams<AT> e{}; e.out = out; e.ldo = vocab; e.scale = 1.0f;
        if (m == 1 && rows_dev == nullptr) {
            GemvRowsParams<AT, WT> p{};
            p.x = x; p.nw = final_norm; p.eps = info.eps; p.w = head; p.K = width; p.O = vocab; p.e = e;
            return this->template launch_gemv<EPI_STORE, NORM_RMS>(st, p);
        }
        NormRowsParams<AT> np{};
        np.x = x; np.ldx = width; np.rows = rows_dev; np.w = final_norm; np.out = hn; np.ldo = width; np.n = width; np.eps = info.eps;
        if (launch_k("rmsnorm_rows_kernel", st, pdl_now, rmsnorm_rows_kernel<AT>, dim3(m), dim3(256), 0, np)) return 1;
        return this->template matmul<EPI_STORE>(st, m, hn, width, head, nullptr, width, vocab, e);
    }

    void set_model_option(const char* name, int value) override {
        if (!strcmp(name, "gla_lanes")) { gla_lanes = value; drop_graphs(); }
    }
    // test access: K and V rows of a parallel layer's attention; a delta-rule layer keeps a state, not rows per position
    int read_kv(cudaStream_t st, uint32_t layer, uint32_t pos0, uint32_t n, float* k_out, float* v_out) override {
        if (layer >= layers.size() || (size_t)pos0 + n > max_tokens) { error = "read_kv: out of range"; return 1; }
        const Layer& L = layers[layer];
        if (L.c.kind != BD_PARALLEL) { error = "read_kv: a delta-rule layer keeps a state, not rows per position"; return 1; }
        GCK(cudaStreamSynchronize(st));
        const size_t nk = (size_t)L.c.G * L.c.dk, nv = (size_t)L.c.G * L.c.dv;
        GCK(cudaMemcpy(k_out, L.kcache + pos0 * nk, n * nk * 4, cudaMemcpyDeviceToHost));
        GCK(cudaMemcpy(v_out, L.vcache + pos0 * nv, n * nv * 4, cudaMemcpyDeviceToHost));
        return 0;
    }
};

ArchModel* badepel_factory(const std::string& dir, const Json& cfg, const ArchOptions& opt, std::string& err) {
    ArchModel* m = nullptr;
    int rc;
    if (opt.dtype == ARCH_F32) {
        auto* g = new BadepelModel<float, float>();
        rc = g->load(dir, cfg, opt);
        m = g;
    } else {
        auto* g = new BadepelModel<__nv_bfloat16, __nv_bfloat16>();
        rc = g->load(dir, cfg, opt);
        m = g;
    }
    if (rc) { err = m->error; delete m; return nullptr; }
    return m;
}

}  // namespace

void register_badepel() { arch_register("Badepel", badepel_factory); }

}  // namespace lmrs
