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
namespace {

using namespace dense;

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
            error = std::string(#call) + ": " + cudaGetErrorString(e_) + " (genetar.cu:" + std::to_string(__LINE__) + ")"; \
            return 1;                                                                                                  \
        }                                                                                                              \
    } while (0)

template <typename AT, typename WT> class GenetarModel : public ArchModel {
  public:
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
    std::vector<void*> owned;   // every device allocation
    WT *embed = nullptr, *bigram = nullptr, *head = nullptr;
    float* final_norm = nullptr;
    uint32_t buckets = 0, mul_prev = 0, mul_cur = 0;
    float logit_scale = 1.0f;
    int width = 0, vocab = 0;
    uint32_t max_tokens = 0;
    int sms = 148;
    uint32_t* d_tokens = nullptr;
    std::map<std::string, std::pair<float*, float*>> rot_tables;
    // scratch, sized for `cap` rows
    size_t cap = 0;
    float *x = nullptr, *qkv = nullptr, *q = nullptr, *gate = nullptr, *vfirst = nullptr, *part = nullptr;
    AT *h = nullptr, *att = nullptr, *act = nullptr, *hn = nullptr;
    uint32_t* d_rows = nullptr;
    float* d_head_tmp = nullptr;
    size_t head_tmp_rows = 0;
    int max_qkv = 0, max_q = 0, max_att = 0, max_ff = 0, max_v = 0, max_H = 0, max_dv = 0;
    static constexpr int MAX_SPLIT = 32;
    bool keep_layers = false;
    float* d_layer_out = nullptr;
    size_t layer_out_rows = 0, layer_out_cap = 0;
    size_t chunk_rows = 2048;
    int use_tc = 1;   // tcgen05 GEMM for aligned bf16 shapes (0: always the CUDA-core kernel)
    DenseGemmCtx gemm_ctx;
    struct GraphEntry { cudaGraphExec_t exec = nullptr; uint64_t kernels = 0; };
    std::map<int, GraphEntry> graphs;   // decode step per position bucket
    std::set<int> warmed;
    const StepParams* graph_step = nullptr;
    // programmatic dependent launch of the decode chain is an option, off by default: measured slower here (1.32 vs 1.14 ms
    // per step at 16 layers of width 2048): the early-launched CTAs of the next kernels sit on the SMs while they wait
    int use_graph = 1, use_pdl = 0;

    ~GenetarModel() override {
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
        if (attn_smem_bytes<4, 8>(c.dk, c.dv, 1) - (size_t)ATT_KT * 32 * 8 * 4 + (size_t)ATT_KT * 32 * ((c.dv + 31) / 32) * 4 > 227 * 1024) {
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
        const std::string k = r.key();
        auto it = rot_tables.find(k);
        if (it == rot_tables.end()) {
            const int half = r.dims / 2;
            std::vector<float> c((size_t)max_tokens * std::max(half, 1)), s(c.size());
            for (int i = 0; i < half; i++) {
                const double f = rot_freq(r, i);
                for (uint32_t p = 0; p < max_tokens; p++) {
                    const double a = (double)p * f;
                    c[(size_t)p * half + i] = (float)cos(a);
                    s[(size_t)p * half + i] = (float)sin(a);
                }
            }
            float *dc = nullptr, *ds = nullptr;
            if (dalloc(&dc, c.size()) || dalloc(&ds, s.size())) return 1;
            GCK(cudaMemcpy(dc, c.data(), c.size() * 4, cudaMemcpyHostToDevice));
            GCK(cudaMemcpy(ds, s.data(), s.size() * 4, cudaMemcpyHostToDevice));
            it = rot_tables.emplace(k, std::make_pair(dc, ds)).first;
        }
        *cos_out = it->second.first;
        *sin_out = it->second.second;
        return 0;
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

    // out = a . w^T with an epilogue; T rows.  One row: the streaming kernel; many rows: tensor cores when the shape
    // allows, else CUDA cores.
    template <int EPI> int matmul(cudaStream_t st, int T, const AT* a, int lda, const WT* w, const WT* w2, int K, int O, const EpiParams<AT>& e) {
        if (T == 1) {
            GemvRowsParams<AT, WT> p{};
            p.a = a; p.w = w; p.w2 = w2; p.K = K; p.O = O; p.e = e;
            return launch_gemv<EPI, false>(st, p);
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
    template <int EPI, bool NORM> int launch_gemv(cudaStream_t st, GemvRowsParams<AT, WT> p) {
        const size_t smem = ((size_t)((p.K + 3) & ~3) + 36 + 2 * 8 + 4) * 4;
        if (optin(gemv_rows_kernel<AT, WT, EPI, NORM>, smem)) return 1;
        const int rows_per_cta = EPI == EPI_GLU ? 8 : 16;
        int grid = (p.O + rows_per_cta - 1) / rows_per_cta;
        // few rows: the warps of a CTA split K instead (two row pairs per CTA)
        p.ksplit = EPI != EPI_GLU && grid < 2 * sms && p.K % Vec16<WT>::N == 0 && p.K >= 1024;
        if (p.ksplit) grid = (p.O + 3) / 4;
        p.pdl = pdl_now ? 1 : 0;
        grid = std::max(1, std::min(grid, sms * 4));
        return launch_k("gemv_rows_kernel", st, pdl_now, gemv_rows_kernel<AT, WT, EPI, NORM>, dim3(grid), dim3(256), smem, p);
    }

    template <int RW, int NI> int launch_attn_t(cudaStream_t st, AttnRowsParams<AT> p, int grid_x, int grid_y) {
        // double-buffered K/V tiles when the head sizes allow 16-byte copies and two CTAs still fit an SM
        p.nbuf = (p.dk % 4 == 0 && p.dv % 4 == 0 && attn_smem_bytes<RW, NI>(p.dk, p.dv, 2) <= 100 * 1024) ? 2 : 1;
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
    int attention(cudaStream_t st, const Layer& L, int T, const PosSrc& ps, uint32_t pos_hint) {
        const LayerCfg& c = L.c;
        const int kv_mul = c.H / c.G;
        AttnRowsParams<AT> p{};
        p.q = q; p.kcache = L.kcache; p.vcache = L.vcache; p.gate = c.rotary ? gate : nullptr; p.out = att; p.part = part;
        p.T = T; p.H = c.H; p.G = c.G; p.dk = c.dk; p.dv = c.dv; p.scale = c.scale; p.softcap = c.softcap; p.ps = ps;
        p.HC = std::min(kv_mul, 16);
        const int chunks = (kv_mul + p.HC - 1) / p.HC;
        int rw = 4;
        if (T == 1) rw = p.HC <= 4 ? 1 : (p.HC <= 8 ? 2 : 4);
        p.TQ = std::max(1, rw * ATT_WARPS / p.HC);
        p.nsplit = 1;
        if (T == 1) {   // decode: split the keys so that the GPU has enough CTAs
            const int tiles = (int)((pos_hint + 1 + ATT_KT - 1) / ATT_KT);
            p.nsplit = std::max(1, std::min({tiles, MAX_SPLIT, (2 * sms) / std::max(1, c.G * chunks)}));
        }
        const int gx = (T + p.TQ - 1) / p.TQ, gy = c.G * chunks;
        int rc = rw == 1 ? launch_attn_rw<1>(st, p, gx, gy) : (rw == 2 ? launch_attn_rw<2>(st, p, gx, gy) : launch_attn_rw<4>(st, p, gx, gy));
        if (rc) return rc;
        if (p.nsplit > 1) {
            AttnCombineParams<AT> cp{};
            cp.part = part; cp.gate = p.gate; cp.out = att; cp.rows = T * c.H; cp.H = c.H; cp.dv = c.dv; cp.nsplit = p.nsplit;
            return launch_k("attn_combine_kernel", st, pdl_now, attn_combine_kernel<AT>, dim3((cp.rows + 3) / 4), dim3(128), 0, cp);
        }
        return 0;
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
                if (launch_gemv<EPI_STORE, true>(st, p)) return 1;
                if (c.has_mlp) {
                    p.w = L.wgate; p.w2 = L.wup; p.O = c.ff; p.e = e_glu;
                    if (launch_gemv<EPI_GLU, true>(st, p)) return 1;
                }
            } else {
                NormRowsParams<AT> np{};
                np.x = x; np.ldx = width; np.w = L.norm1; np.out = h; np.ldo = width; np.n = width; np.eps = info.eps;
                rmsnorm_rows_kernel<AT><<<T, 256, 0, st>>>(np);
                if (check_launch("rmsnorm_rows_kernel")) return 1;
                if (matmul<EPI_STORE>(st, T, h, width, L.wqkv, nullptr, width, L.qkv_rows, e_qkv)) return 1;
                if (c.has_mlp && matmul<EPI_GLU>(st, T, h, width, L.wgate, L.wup, width, c.ff, e_glu)) return 1;
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
            if (matmul<EPI_RESID>(st, T, att, c.H * c.dv, L.wo, nullptr, c.H * c.dv, width, e_res)) return 1;
            if (c.has_mlp) {
                e_res.ls = L.ls2;
                if (matmul<EPI_RESID>(st, T, act, c.ff, L.wdown, nullptr, c.ff, width, e_res)) return 1;
            }
            if (keep_layers && d_layer_out && (size_t)T == layer_out_rows)
                GCK(cudaMemcpyAsync(d_layer_out + li * (size_t)T * width, x, (size_t)T * width * 4, cudaMemcpyDeviceToDevice, st));
        }
        return 0;
    }
    // final norm + head over `m` rows of x given by d_rows[0..m) -> out [m][vocab]
    int head_rows(cudaStream_t st, int m, const uint32_t* rows_dev, float* out) {
        EpiParams<AT> e{}; e.out = out; e.ldo = vocab; e.scale = logit_scale;
        if (m == 1 && rows_dev == nullptr) {
            GemvRowsParams<AT, WT> p{};
            p.x = x; p.nw = final_norm; p.eps = info.eps; p.w = head; p.K = width; p.O = vocab; p.e = e;
            return launch_gemv<EPI_STORE, true>(st, p);
        }
        NormRowsParams<AT> np{};
        np.x = x; np.ldx = width; np.rows = rows_dev; np.w = final_norm; np.out = hn; np.ldo = width; np.n = width; np.eps = info.eps;
        rmsnorm_rows_kernel<AT><<<m, 256, 0, st>>>(np);
        if (check_launch("rmsnorm_rows_kernel")) return 1;
        return matmul<EPI_STORE>(st, m, hn, width, head, nullptr, width, vocab, e);
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
        if (ensure_scratch(std::min(n, chunk_rows))) return 1;
        if (keep_layers) {
            layer_out_rows = n <= chunk_rows ? n : 0;
            if (layer_out_rows && layers.size() * n * width > layer_out_cap) {
                dfree(d_layer_out); d_layer_out = nullptr; layer_out_cap = 0;
                if (dalloc(&d_layer_out, layers.size() * n * width)) return 1;
                layer_out_cap = layers.size() * n * width;
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
        const size_t n = layers.size() * layer_out_rows * width;
        if (!keep_layers || !d_layer_out || n == 0) { error = "no layer outputs were kept"; return 1; }
        if (capacity < n) { error = "buffer too small for the layer outputs"; return 1; }
        GCK(cudaStreamSynchronize(st));
        GCK(cudaMemcpy(out, d_layer_out, n * 4, cudaMemcpyDeviceToHost));
        *n_floats = n;
        return 0;
    }
    void set_keep_layer_outputs(bool on) override { keep_layers = on; }
    int read_kv(cudaStream_t st, uint32_t layer, uint32_t pos0, uint32_t n, float* k_out, float* v_out) override {
        if (layer >= layers.size() || (size_t)pos0 + n > max_tokens) { error = "read_kv: out of range"; return 1; }
        const Layer& L = layers[layer];
        const size_t nk = (size_t)L.c.G * L.c.dk, nv = (size_t)L.c.G * L.c.dv;
        GCK(cudaStreamSynchronize(st));
        GCK(cudaMemcpy(k_out, L.kcache + pos0 * nk, n * nk * 4, cudaMemcpyDeviceToHost));
        GCK(cudaMemcpy(v_out, L.vcache + pos0 * nv, n * nv * 4, cudaMemcpyDeviceToHost));
        return 0;
    }
    void set_option(const char* name, int value) override {
        if (!strcmp(name, "chunk_rows")) chunk_rows = (size_t)std::max(1, value);
        else if (!strcmp(name, "tensor_cores")) use_tc = value;
        else if (!strcmp(name, "graphs")) { use_graph = value; if (!value) drop_graphs(); }
        else if (!strcmp(name, "pdl")) { use_pdl = value; drop_graphs(); }
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
