// genetar.cu -- the Genetar architecture (arch.h): a decoder whose layers are PARALLEL blocks,
//     h = rmsnorm(x, norm1);   x <- x + ls1 * mixer(h) + ls2 * ff(h)
// with two kinds of attention mixer listed per layer in config.json "layers":
//   "attention"    q and k heads divided by their root mean square (no weight), no positional rotation
//   "attention_2"  partial rotary on the first rot.dims dimensions (rotate-half pairing, optional Llama-3.1 style
//                  frequency scaling), and a per-head sigmoid output gate computed from h
// both with grouped KV heads, score scale and tanh soft-cap from the config, causal softmax, and "value mixing": the
// values of every v_mix layer but the first are blended with the first such layer's values of the same token before they
// are cached.  The input embedding adds a hashed bigram row of (previous token, token); the feed-forward is a SiLU GLU;
// the logits are head(rmsnorm(x, final.norm)) * logit_scale.
// Everything model-specific comes from config.json and the tensor shapes; the kernels are the generic ones of
// dense_ops.cuh / dense_gemm.cuh.  Two operand modes: bf16 weights and activations with f32 accumulation (residual,
// norms, scores, softmax, angles stay f32), or f32 everywhere.  The KV cache is f32 [max_tokens][kv_heads * dim] per
// layer, addressed by position like the cache of the LMRS models; the token history (for the bigram row) sits beside it.
#include "dense_model.cuh"

namespace lmrs {
namespace {

struct RotCfg {
    int dims = 0;
    double base = 10000.0;
    bool scaled = false;
    double factor = 1.0, low = 1.0, high = 1.0, original = 1.0;
    std::string key() const {
        char b[256];
        snprintf(b, sizeof b, "%d/%.17g/%d/%.17g/%.17g/%.17g/%.17g", dims, base, (int)scaled, factor, low, high, original);
        return b;
    }
};
struct LayerCfg {
    bool rotary = false;   // "attention_2": rotary + head gate; "attention": unit-norm q/k
    int H = 0, G = 0, dk = 0, dv = 0;
    float scale = 1.0f, softcap = 0.0f;
    bool v_mix = false;
    RotCfg rot;
    bool has_mlp = false;
    int ff = 0;
};

// frequency of rotary pair i (angle = position * f_i), with the piecewise wavelength-dependent rescaling when configured
static double rot_freq(const RotCfg& r, int i) {
    const double kPi = 3.14159265358979323846;
    double f = pow(r.base, -2.0 * (double)i / (double)r.dims);
    if (r.scaled) {
        const double wl = 2.0 * kPi / f;
        if (wl > r.original / r.low) f = f / r.factor;                  // long wavelengths: slowed down by `factor`
        else if (!(wl < r.original / r.high)) {                          // in between: blend
            const double s = (r.original / wl - r.low) / (r.high - r.low);
            f = (1.0 - s) * f / r.factor + s * f;
        }
    }
    return f;
}

template <typename AT, typename WT> class GenetarModel : public DenseModel<AT, WT> {
  public:
    typedef DenseModel<AT, WT> B;
    using B::error; using B::launches; using B::info; using B::d_logits; using B::owned; using B::width; using B::vocab;
    using B::max_tokens; using B::sms; using B::d_tokens; using B::cap; using B::x; using B::hn; using B::d_rows; using B::MAX_SPLIT;
    using B::keep_layers; using B::gemm_ctx; using B::pdl_now; using B::dalloc; using B::dfree; using B::need; using B::upload_w;
    using B::upload_f32; using B::check_launch; using B::launch_k; using B::drop_graphs;
    struct Layer {
        LayerCfg c;
        WT *wqkv = nullptr, *wo = nullptr, *wgate = nullptr, *wup = nullptr, *wdown = nullptr;
        float *norm1 = nullptr, *ls1 = nullptr, *ls2 = nullptr, *vmix = nullptr;
        float *kcache = nullptr, *vcache = nullptr;
        const float *rot_cos = nullptr, *rot_sin = nullptr;
        int qkv_rows = 0;   // H*dk + G*dk + G*dv (+ H gate rows)
        int v_mode = V_PLAIN;
    };
    std::vector<Layer> layers;
    WT *embed = nullptr, *bigram = nullptr, *head = nullptr;
    float* final_norm = nullptr;
    uint32_t buckets = 0, mul_prev = 0, mul_cur = 0;
    float logit_scale = 1.0f;
    // scratch, sized for `cap` rows
    float *qkv = nullptr, *q = nullptr, *gate = nullptr, *vfirst = nullptr, *part = nullptr;
    AT *h = nullptr, *att = nullptr, *act = nullptr;
    int max_qkv = 0, max_q = 0, max_att = 0, max_ff = 0, max_v = 0, max_H = 0, max_dv = 0;

    size_t n_layers() const override { return layers.size(); }

    int parse_layer(const Json& jl, size_t li, LayerCfg& c) {
        const std::string type = jl.at("type").str;
        const std::string where = "config.json layers[" + std::to_string(li) + "]";
        if (type == "attention") c.rotary = false;
        else if (type == "attention_2") c.rotary = true;
        else { error = where + ": unknown layer type '" + type + "'"; return 1; }
        const Json& m = jl.at("mixer");
        c.H = (int)m.at("heads").number(0); c.G = (int)m.at("kv_heads").number(c.H);
        c.dk = (int)m.at("dim").number(0); c.dv = (int)m.at("vdim").number(c.dk);
        c.scale = (float)m.at("scale").number(1.0);
        c.softcap = m.has("softcap") ? (float)m.at("softcap").number(0.0) : 0.0f;
        c.v_mix = m.has("v_mix") && m.at("v_mix").truth();
        if (c.H <= 0 || c.G <= 0 || c.dk <= 0 || c.dv <= 0 || c.H % c.G != 0) { error = where + ": bad head geometry"; return 1; }
        if (c.dv > 256) { error = where + ": vdim above 256 is not supported by the attention kernel"; return 1; }
        if (!B::attention_fits(c.dk, c.dv)) {
            error = where + ": head dim " + std::to_string(c.dk) + " needs more shared memory than an SM has for the attention tiles";
            return 1;
        }
        if (c.rotary) {
            const Json& r = m.at("rot");
            if (!r.is_obj()) { error = where + ": attention_2 without 'rot'"; return 1; }
            c.rot.dims = (int)r.at("dims").number(c.dk);
            c.rot.base = r.at("base").number(10000.0);
            if (c.rot.dims < 0 || c.rot.dims > c.dk || c.rot.dims % 2 != 0) { error = where + ": rot.dims must be even and at most dim"; return 1; }
            if (r.has("scaling")) {
                const Json& s = r.at("scaling");
                c.rot.scaled = true;
                c.rot.factor = s.at("factor").number(1.0); c.rot.low = s.at("low").number(1.0);
                c.rot.high = s.at("high").number(4.0); c.rot.original = s.at("original").number(8192.0);
            }
        }
        if (jl.has("mlp")) {
            const Json& f = jl.at("mlp");
            const std::string kind = f.has("kind") ? f.at("kind").str : "dense";
            if (kind != "dense") { error = where + ": unknown mlp kind '" + kind + "'"; return 1; }
            c.has_mlp = true;
            c.ff = (int)f.at("ff").number(0);
            if (c.ff <= 0) { error = where + ": mlp.ff missing"; return 1; }
        }
        return 0;
    }

    int rot_table(const RotCfg& r, const float** cos_out, const float** sin_out) {
        std::vector<double> f;
        for (int i = 0; i < r.dims / 2; i++) f.push_back(rot_freq(r, i));
        return this->angle_tables(r.key(), f, 1.0, cos_out, sin_out);
    }

    int load(const std::string& dir, const Json& cfg, const ArchOptions& opt) {
        sms = opt.sms;
        gemm_ctx.sms = opt.sms;
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
        if (cfg.at("embedding").has("bigram")) {
            const Json& b = cfg.at("embedding").at("bigram");
            const double nb = b.at("buckets").number(0);
            if (!(nb >= 1.0 && nb < 2147483648.0)) { error = "config.json: embedding.bigram.buckets must be a positive 31-bit number"; return 1; }
            buckets = (uint32_t)nb;
            // (prev * a + cur * b) mod m only needs a and b modulo m: reduced here, the products on the device stay below 2^63
            auto mod_m = [&](double v) { return (uint32_t)((unsigned long long)fabs(v) % buckets); };
            if (b.at("mul_prev").number(0) < 0 || b.at("mul_cur").number(0) < 0) { error = "config.json: negative bigram multipliers are not supported"; return 1; }
            mul_prev = mod_m(b.at("mul_prev").number(0));
            mul_cur = mod_m(b.at("mul_cur").number(0));
            if (need(st, "bigram", {(int64_t)buckets + 1, width}, &t) || dalloc(&bigram, t->numel()) || upload_w(t, bigram)) return 1;
        }
        if (need(st, "head", {vocab, width}, &t) || dalloc(&head, t->numel()) || upload_w(t, head)) return 1;
        if (need(st, "final.norm", {width}, &t) || upload_f32(t, &final_norm)) return 1;
        layers.resize(jl.arr.size());
        int first_vmix = -1;
        for (size_t li = 0; li < layers.size(); li++) {
            Layer& L = layers[li];
            if (parse_layer(jl.arr[li], li, L.c)) return 1;
            const LayerCfg& c = L.c;
            const std::string p = "l" + std::to_string(li) + ".";
            const int nq = c.H * c.dk, nk = c.G * c.dk, nv = c.G * c.dv;
            L.qkv_rows = nq + nk + nv + (c.rotary ? c.H : 0);
            if (dalloc(&L.wqkv, (size_t)L.qkv_rows * width)) return 1;
            if (need(st, p + "mix.q", {nq, width}, &t) || upload_w(t, L.wqkv)) return 1;
            if (need(st, p + "mix.k", {nk, width}, &t) || upload_w(t, L.wqkv + (size_t)nq * width)) return 1;
            if (need(st, p + "mix.v", {nv, width}, &t) || upload_w(t, L.wqkv + (size_t)(nq + nk) * width)) return 1;
            if (c.rotary && (need(st, p + "mix.g", {c.H, width}, &t) || upload_w(t, L.wqkv + (size_t)(nq + nk + nv) * width))) return 1;
            if (need(st, p + "mix.o", {width, c.H * c.dv}, &t) || dalloc(&L.wo, t->numel()) || upload_w(t, L.wo)) return 1;
            if (need(st, p + "norm1", {width}, &t) || upload_f32(t, &L.norm1)) return 1;
            if (need(st, p + "ls1", {width}, &t) || upload_f32(t, &L.ls1)) return 1;
            if (c.v_mix) {
                if (first_vmix < 0) { first_vmix = (int)li; L.v_mode = V_FIRST; }
                else {
                    L.v_mode = V_MIX;
                    if (nv != layers[first_vmix].c.G * layers[first_vmix].c.dv) { error = "layers that mix values must have equally sized values"; return 1; }
                    t = st.find(p + "mix.vmix");
                    if (!t || t->numel() != 1 || (t->dtype != "BF16" && t->dtype != "F32")) { error = "tensor '" + p + "mix.vmix' must hold one number"; return 1; }
                    if (upload_f32(t, &L.vmix)) return 1;
                }
            }
            if (c.has_mlp) {
                if (need(st, p + "mlp.gate", {c.ff, width}, &t) || dalloc(&L.wgate, t->numel()) || upload_w(t, L.wgate)) return 1;
                if (need(st, p + "mlp.up", {c.ff, width}, &t) || dalloc(&L.wup, t->numel()) || upload_w(t, L.wup)) return 1;
                if (need(st, p + "mlp.down", {width, c.ff}, &t) || dalloc(&L.wdown, t->numel()) || upload_w(t, L.wdown)) return 1;
                if (need(st, p + "ls2", {width}, &t) || upload_f32(t, &L.ls2)) return 1;
            }
            if (dalloc(&L.kcache, (size_t)max_tokens * nk) || dalloc(&L.vcache, (size_t)max_tokens * nv)) return 1;
            if (c.rotary && rot_table(c.rot, &L.rot_cos, &L.rot_sin)) return 1;
            max_qkv = std::max(max_qkv, L.qkv_rows); max_q = std::max(max_q, nq); max_att = std::max(max_att, c.H * c.dv);
            max_ff = std::max(max_ff, c.ff); max_v = std::max(max_v, nv); max_H = std::max(max_H, c.H); max_dv = std::max(max_dv, c.dv);
        }
        if (dalloc(&d_tokens, (size_t)max_tokens) || dalloc(&d_logits, (size_t)vocab)) return 1;
        GCK(cudaMemset(d_tokens, 0, (size_t)max_tokens * 4));
        info.architecture = "Genetar";
        info.vocab = (uint32_t)vocab; info.width = (uint32_t)width; info.n_layers = (uint32_t)layers.size(); info.max_tokens = max_tokens;
        info.heads = (uint32_t)layers[0].c.H; info.kv_heads = (uint32_t)layers[0].c.G; info.head_dim = (uint32_t)layers[0].c.dk;
        info.ff = (uint32_t)layers[0].c.ff; info.dtype = opt.dtype; info.eps = eps;
        if (ensure_scratch(1)) return 1;
        return 0;
    }

    int ensure_scratch(size_t rows) {
        if (rows <= cap) return 0;
        drop_graphs();   // captured launches point into the old scratch
        for (void* p : {(void*)x, (void*)qkv, (void*)q, (void*)gate, (void*)vfirst, (void*)part, (void*)h, (void*)att, (void*)act, (void*)hn, (void*)d_rows}) dfree(p);
        cap = 0;
        if (dalloc(&x, rows * width) || dalloc(&qkv, rows * max_qkv) || dalloc(&q, rows * max_q) || dalloc(&gate, rows * max_H) ||
            dalloc(&vfirst, rows * max_v) || dalloc(&h, rows * width) || dalloc(&att, rows * max_att) ||
            dalloc(&act, rows * std::max(max_ff, 1)) || dalloc(&hn, rows * width) || dalloc(&d_rows, rows) ||
            dalloc(&part, (size_t)max_H * MAX_SPLIT * (max_dv + 2)))
            return 1;
        cap = rows;
        return 0;
    }

    int attention(cudaStream_t st, const Layer& L, int T, const PosSrc& ps, uint32_t pos_hint) {
        const LayerCfg& c = L.c;
        AttnRowsParams<AT> p{};
        p.q = q; p.kcache = L.kcache; p.vcache = L.vcache; p.gate = c.rotary ? gate : nullptr; p.out = att;
        p.T = T; p.H = c.H; p.G = c.G; p.dk = c.dk; p.dv = c.dv; p.scale = c.scale; p.softcap = c.softcap; p.ps = ps;
        p.k_ld = c.G * c.dk; p.v_ld = c.G * c.dv;
        return this->attention_launch(st, p, part, pos_hint);
    }

    // the layers over T rows at positions pos ..; x holds the residual stream on return
    int run_layers(cudaStream_t st, int T, const PosSrc& ps, uint32_t pos_hint) {
        {
            EmbedRowsParams<WT> p{};
            p.embed = embed; p.bigram = bigram; p.tokens = d_tokens; p.x = x; p.width = width; p.ps = ps;
            p.buckets = buckets; p.mul_prev = mul_prev; p.mul_cur = mul_cur;
            embed_rows_kernel<WT><<<T, 128, 0, st>>>(p);
            if (check_launch("embed_rows_kernel")) return 1;
        }
        for (size_t li = 0; li < layers.size(); li++) {
            const Layer& L = layers[li];
            const LayerCfg& c = L.c;
            EpiParams<AT> e_qkv{}; e_qkv.out = qkv; e_qkv.ldo = L.qkv_rows; e_qkv.scale = 1.0f;
            EpiParams<AT> e_glu{}; e_glu.act = act; e_glu.lda = c.ff;
            if (T == 1) {   // the norm is a prologue of the streaming kernels; both read x before any epilogue adds to it
                GemvRowsParams<AT, WT> p{};
                p.x = x; p.nw = L.norm1; p.eps = info.eps; p.w = L.wqkv; p.K = width; p.O = L.qkv_rows; p.e = e_qkv;
                if (this->template launch_gemv<EPI_STORE, NORM_RMS>(st, p)) return 1;
                if (c.has_mlp) {
                    p.w = L.wgate; p.w2 = L.wup; p.O = c.ff; p.e = e_glu;
                    if (this->template launch_gemv<EPI_GLU, NORM_RMS>(st, p)) return 1;
                }
            } else {
                NormRowsParams<AT> np{};
                np.x = x; np.ldx = width; np.w = L.norm1; np.out = h; np.ldo = width; np.n = width; np.eps = info.eps;
                rmsnorm_rows_kernel<AT><<<T, 256, 0, st>>>(np);
                if (check_launch("rmsnorm_rows_kernel")) return 1;
                if (this->template matmul<EPI_STORE>(st, T, h, width, L.wqkv, nullptr, width, L.qkv_rows, e_qkv)) return 1;
                if (c.has_mlp && this->template matmul<EPI_GLU>(st, T, h, width, L.wgate, L.wup, width, c.ff, e_glu)) return 1;
            }
            {
                QkvPostParams p{};
                p.qkv = qkv; p.ld = L.qkv_rows; p.H = c.H; p.G = c.G; p.dk = c.dk; p.dv = c.dv;
                p.qk_mode = c.rotary ? (c.rot.dims > 0 ? QK_ROTARY : QK_PLAIN) : QK_UNITNORM; p.eps = info.eps;
                p.rot_dims = c.rot.dims; p.rot_cos = L.rot_cos; p.rot_sin = L.rot_sin;
                p.v_mode = L.v_mode; p.v_first = vfirst; p.lambda = L.vmix; p.has_gate = c.rotary;
                p.q_out = q; p.gate_out = gate; p.kcache = L.kcache; p.vcache = L.vcache; p.ps = ps;
                const int tasks = c.H + c.G + (c.G * c.dv + 127) / 128 + 1;
                const dim3 grid(T, T >= 64 ? std::min(4, (tasks + 3) / 4) : std::min(16, (tasks + 3) / 4));
                if (launch_k("qkv_post_kernel", st, pdl_now, qkv_post_kernel, grid, dim3(128), 0, p)) return 1;
            }
            if (attention(st, L, T, ps, pos_hint)) return 1;
            EpiParams<AT> e_res{}; e_res.out = x; e_res.ldo = width; e_res.ls = L.ls1;
            if (this->template matmul<EPI_RESID>(st, T, att, c.H * c.dv, L.wo, nullptr, c.H * c.dv, width, e_res)) return 1;
            if (c.has_mlp) {
                e_res.ls = L.ls2;
                if (this->template matmul<EPI_RESID>(st, T, act, c.ff, L.wdown, nullptr, c.ff, width, e_res)) return 1;
            }
            if (this->keep_layer(st, li, T)) return 1;
        }
        return 0;
    }
    // final norm + head over `m` rows of x given by d_rows[0..m) -> out [m][vocab]
    int head_rows(cudaStream_t st, int m, const uint32_t* rows_dev, float* out) {
        EpiParams<AT> e{}; e.out = out; e.ldo = vocab; e.scale = logit_scale;
        if (m == 1 && rows_dev == nullptr) {
            GemvRowsParams<AT, WT> p{};
            p.x = x; p.nw = final_norm; p.eps = info.eps; p.w = head; p.K = width; p.O = vocab; p.e = e;
            return this->template launch_gemv<EPI_STORE, NORM_RMS>(st, p);
        }
        NormRowsParams<AT> np{};
        np.x = x; np.ldx = width; np.rows = rows_dev; np.w = final_norm; np.out = hn; np.ldo = width; np.n = width; np.eps = info.eps;
        rmsnorm_rows_kernel<AT><<<m, 256, 0, st>>>(np);
        if (check_launch("rmsnorm_rows_kernel")) return 1;
        return this->template matmul<EPI_STORE>(st, m, hn, width, head, nullptr, width, vocab, e);
    }

    int read_kv(cudaStream_t st, uint32_t layer, uint32_t pos0, uint32_t n, float* k_out, float* v_out) override {
        if (layer >= layers.size() || (size_t)pos0 + n > max_tokens) { error = "read_kv: out of range"; return 1; }
        const Layer& L = layers[layer];
        const size_t nk = (size_t)L.c.G * L.c.dk, nv = (size_t)L.c.G * L.c.dv;
        GCK(cudaStreamSynchronize(st));
        GCK(cudaMemcpy(k_out, L.kcache + pos0 * nk, n * nk * 4, cudaMemcpyDeviceToHost));
        GCK(cudaMemcpy(v_out, L.vcache + pos0 * nv, n * nv * 4, cudaMemcpyDeviceToHost));
        return 0;
    }
};

ArchModel* genetar_factory(const std::string& dir, const Json& cfg, const ArchOptions& opt, std::string& err) {
    ArchModel* m = nullptr;
    int rc;
    if (opt.dtype == ARCH_F32) {
        auto* g = new GenetarModel<float, float>();
        rc = g->load(dir, cfg, opt);
        m = g;
    } else {
        auto* g = new GenetarModel<__nv_bfloat16, __nv_bfloat16>();
        rc = g->load(dir, cfg, opt);
        m = g;
    }
    if (rc) { err = m->error; delete m; return nullptr; }
    return m;
}

}  // namespace

// called by the handle code before the first arch_open: a static registrar in a library TU that nothing references could
// be dropped by the linker, an explicit call cannot
void register_genetar() { arch_register("Genetar", genetar_factory); }

}  // namespace lmrs
