// Mulenex: a decoder-only design on one fp32 residual with a norm on both sides of every sublayer, whose mixers are a
// matrix-memory recurrence with exponential gating (mLSTM) or softmax attention without rotation, and whose feed-forward
// is a squared-ReLU layer with biases, a mixture of SiLU-gated experts with a shared expert, or nothing.
//
//   x[t]     = embed[token] + sinusoid(position)                                              (hyper.cu embed_sinusoid)
//   sublayer : x <- x + N_post(f(N_pre(x))),  N(u) = u / sqrt(mean(u^2) + eps) * (1 + w)        (hyper.cu sandwich_step)
//   mlstm    : per head C [dim, vdim], n [dim], m:  i = cap tanh((W_i h + b_i) / cap),  f = logsigmoid(cap tanh((W_f h + b_f) / cap)),
//              m_t = max(f + m_(t-1), i),  C_t = e^(f + m_(t-1) - m_t) C + e^(i - m_t) k v^T,  n_t likewise with k,
//              o = C_t^T q / (max(|n_t . q|, e^(-m_t)) + 1e-6),  q scaled by dim^(-1/2); per head o / rms(o), all heads times a
//              weight, times sigmoid(W_g h), then W_o                          (gla.cu: mlstm_gates, gla_scan, recurrent_out_gate)
//   attention: grouped key/value heads; q and k of every head RMS-normed with a weight shared by the heads; no rotation;
//              q times 1 + coef ln(floor((p + 1) / every) + 1); score = cap tanh(scale q.k / cap); causal softmax; in every
//              value-blending layer but the first, v <- (1 - lambda) v + lambda v_first (the first blending layer's values of
//              the same token), and the blended v is what the cache holds; head h's output times sigmoid(W_g h)_h; W_o
//                                                                                              (window_attention.cu)
//   dense ff : W_down relu(W_up h + b_up)^2 + b_down                                           (linear.cu, norm_act.cu)
//   moe ff   : z = W_r h + b_r in fp32; the `top` largest z, weights = softmax over those z alone; expert(h) = W_down
//              (silu(W_gate h) * (W_up h)); plus sigmoid(w_sg . h) * shared(h)                  (moe.cu, linear.cu)
//   logits   = head N_final(x)
//
// Per layer the kernel sequence is: the boundary (previous write-back with its post-norm, this sublayer's pre-norm), ONE
// input projection for everything that reads the mixer's normed input (q, k, v and the gate rows concatenated row-wise at
// load), the mixer, the output projection, the boundary, the feed-forward.  Every size and constant comes from
// config.json; matrices and activations are bf16 or fp32, with the residual, norms, softmax, router, gates of the
// recurrence and its state in fp32 either way.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <string.h>

#include <algorithm>

#include "errors.h"
#include "gemm.h"
#include "model.h"

namespace b200 {
namespace {

typedef __nv_bfloat16 bf16;

enum MixerKind { MIX_ATTENTION = 0, MIX_MLSTM = 1 };
enum MlpKind { MLP_NONE = 0, MLP_DENSE = 1, MLP_MOE = 2 };

struct LayerSpec {
  int mixer = MIX_ATTENTION;
  int heads = 0, kv_heads = 0, dim = 0, vdim = 0;
  // attention
  float scale = 1.f, softcap = 0.f, qt_coef = 0.f;
  int qt_every = 0;
  bool v_mix = false, v_first = false;   // blends its values / is the first layer that does (its values are the ones blended in)
  // mlstm
  float gate_cap = 0.f;
  // feed-forward
  int mlp = MLP_NONE;
  int ff = 0;                              // dense width, or one expert's
  int experts = 0, top = 0, sff = 0;
  bool shared = false;
  // column layout of the input projection's output row
  int n_in = 0, off_q = 0, off_k = 0, off_v = 0, off_g = 0;
  int k_out = 0, n_sh = 0;
};

struct LayerWeights {
  void* w_in = nullptr;     // [n_in, width]
  void* w_out = nullptr;    // [width, k_out]
  float *norm1 = nullptr, *norm1b = nullptr, *norm2 = nullptr, *norm2b = nullptr;   // 1 + stored weight
  float *q_norm = nullptr, *k_norm = nullptr;   // attention: [dim]
  float v_lambda = 0.f;                         // attention: blending weight
  void* w_gates = nullptr;  // mlstm: [2 heads, width], input-gate rows then forget-gate rows
  float* b_gates = nullptr; // mlstm: [2 heads]
  float* h_norm = nullptr;  // mlstm: [heads * vdim]
  void *up = nullptr, *down = nullptr;          // dense: [ff, width], [width, ff]
  float *up_b = nullptr, *down_b = nullptr;
  void* router = nullptr;   // [experts (+ 1), width]: the router rows, then the shared expert's gate row
  float* router_b = nullptr;   // [experts (+ 1)], 0 for the shared gate
  void* e_gu = nullptr;     // [experts][2 ff][width]  gate rows, then up rows
  void* e_down = nullptr;   // [experts][width][ff]
  void* sh_in = nullptr;    // [n_sh, width]: gate [sff] | up [sff]
  void* sh_down = nullptr;  // [width, sff]
  void* cache = nullptr;    // attention: [num_blocks * page][kv_heads * (dim + vdim)]
  float* state = nullptr;   // mlstm: [slots][heads][dim][vdim]
  float* nstate = nullptr;  // mlstm: [slots][heads][dim], the normaliser
  float* mstate = nullptr;  // mlstm: [slots][heads], the log-scale
  GemmPlan p_in, p_out, p_up, p_down, p_shin, p_shdown;
  std::vector<GemmPlan> p_egu, p_edown;
  CUtensorMap xm_out[kGemmNumBlockN], xm_ffh[kGemmNumBlockN], xm_shact[kGemmNumBlockN];
  bool tc_in = false, tc_out = false, tc_up = false, tc_down = false, tc_shin = false, tc_shdown = false;
};

bool jnum(const JVal* o, const char* k, double* out) {
  const JVal* v = o ? o->get(k) : nullptr;
  if (!v || v->type != JVal::Num) return false;
  *out = v->num;
  return true;
}

class Mulenex : public Model {
 public:
  DType dt;
  int V = 0, W = 0;
  float eps = 1e-5f;
  std::vector<LayerSpec> spec;
  std::vector<LayerWeights> wts;
  ModelEnv env;
  void *embed = nullptr, *head = nullptr;
  float* fin_w = nullptr;
  float2* pos_freq = nullptr;
  // activations
  float* x = nullptr;            // [Tcap][W]
  void *h = nullptr, *inb = nullptr, *ycat = nullptr, *ao = nullptr, *fo = nullptr, *hrow = nullptr, *vfirst = nullptr, *ffh = nullptr;
  void *egu = nullptr, *eact = nullptr, *sh = nullptr, *shact = nullptr, *sdown = nullptr;
  float *qn = nullptr, *o32 = nullptr, *gpre = nullptr, *gkeep = nullptr, *gtake = nullptr, *gfloor = nullptr, *gnq = nullptr;
  float *scores = nullptr, *topw = nullptr, *edown = nullptr, *logits = nullptr;
  int *topi = nullptr, *sorted_rows = nullptr, *tile_group = nullptr, *pair_pos = nullptr, *iota = nullptr;
  int row_cap = 0, moe_cap = 0, vfirst_ld = 0;
  void *hsorted = nullptr, *edown16 = nullptr;
  int *expert_rows = nullptr, *expert_rows_host = nullptr;
  std::vector<void*> allocs;
  float* gemm_ws = nullptr;
  int* gemm_counters = nullptr;
  CUtensorMap xm_h[kGemmNumBlockN];
  bool use_tc = false;

  explicit Mulenex(DType d) : dt(d) {}
  ~Mulenex() override {
    for (auto& w : wts) {
      if (w.tc_in) gemm_plan_destroy(&w.p_in);
      if (w.tc_out) gemm_plan_destroy(&w.p_out);
      if (w.tc_up) gemm_plan_destroy(&w.p_up);
      if (w.tc_down) gemm_plan_destroy(&w.p_down);
      if (w.tc_shin) gemm_plan_destroy(&w.p_shin);
      if (w.tc_shdown) gemm_plan_destroy(&w.p_shdown);
      for (auto& p : w.p_egu) gemm_plan_destroy(&p);
      for (auto& p : w.p_edown) gemm_plan_destroy(&p);
    }
    if (expert_rows_host) cudaFreeHost(expert_rows_host);
    for (void* p : allocs) cudaFree(p);
  }
  const char* arch() const override { return "Mulenex"; }
  int vocab() const override { return V; }

  size_t cache_bytes_per_block(int page) const override {
    size_t b = 0;
    for (auto& s : spec)
      if (s.mixer == MIX_ATTENTION) b += static_cast<size_t>(page) * s.kv_heads * (s.dim + s.vdim) * dtype_bytes(dt);
    return b;
  }
  size_t state_bytes_per_slot() const override {
    size_t b = 0;
    for (auto& s : spec)
      if (s.mixer == MIX_MLSTM) b += (static_cast<size_t>(s.heads) * s.dim * (s.vdim + 1) + s.heads) * sizeof(float);   // C, n, m
    return b;
  }
  // every attention layer sees the whole sequence: no page is ever behind all windows
  int cache_window() const override { return 0; }

  // ------------------------------------------------------------ config.json
  bool parse(const JVal& c, std::string* err) {
    double d = 0;
    auto whole = [&](const JVal* o, const char* k, int lo, int* out, const std::string& where) {
      double v = 0;
      if (!jnum(o, k, &v) || v < lo || v != floor(v) || v > 2147483647.0) { *err = "config: " + where + k; return false; }
      *out = static_cast<int>(v);
      return true;
    };
    if (!whole(&c, "vocab", 1, &V, "") || !whole(&c, "width", 1, &W, "")) return false;
    if (jnum(c.get("norm"), "eps", &d)) eps = static_cast<float>(d);
    const JVal* ls = c.get("layers");
    if (!ls || ls->type != JVal::Arr || ls->arr.empty()) { *err = "config: layers"; return false; }
    int first_blend = -1;
    for (size_t i = 0; i < ls->arr.size(); ++i) {
      const JVal& L = ls->arr[i];
      const std::string where = "layer " + std::to_string(i) + " ";
      LayerSpec s;
      const JVal* ty = L.get("type");
      if (!ty || ty->type != JVal::Str) { *err = "config: " + where + "type"; return false; }
      const JVal* mx = L.get("mixer");
      if (!mx || mx->type != JVal::Obj) { *err = "config: " + where + "mixer"; return false; }
      if (!whole(mx, "heads", 1, &s.heads, where + "mixer.") || !whole(mx, "dim", 1, &s.dim, where + "mixer.") ||
          !whole(mx, "vdim", 1, &s.vdim, where + "mixer.")) return false;
      if (ty->str == "attention") {
        s.mixer = MIX_ATTENTION;
        s.kv_heads = s.heads;
        if (mx->get("kv_heads") && !whole(mx, "kv_heads", 1, &s.kv_heads, where + "mixer.")) return false;
        if (s.heads % s.kv_heads) { *err = "config: " + where + "mixer.heads is no multiple of kv_heads"; return false; }
        if (s.vdim > 256) { *err = "config: " + where + "mixer.vdim above 256"; return false; }
        s.scale = 1.0f / sqrtf(static_cast<float>(s.dim));
        if (jnum(mx, "scale", &d)) s.scale = static_cast<float>(d);
        if (jnum(mx, "softcap", &d) && d > 0) s.softcap = static_cast<float>(d);
        if (const JVal* qt = mx->get("q_temp")) {
          if (qt->type == JVal::Obj) {
            if (!jnum(qt, "coef", &d)) { *err = "config: " + where + "mixer.q_temp.coef"; return false; }
            s.qt_coef = static_cast<float>(d);
            if (!whole(qt, "every", 1, &s.qt_every, where + "mixer.q_temp.")) return false;
          }
        }
        const JVal* vm = mx->get("v_mix");
        s.v_mix = vm && vm->type == JVal::Bool && vm->b;
        if (s.v_mix) {
          if (first_blend < 0) { first_blend = static_cast<int>(i); s.v_first = true; }
          else if (spec[first_blend].kv_heads != s.kv_heads || spec[first_blend].vdim != s.vdim) {
            *err = "config: " + where + "blends values of another shape than layer " + std::to_string(first_blend) + "'s";
            return false;
          }
        }
      } else if (ty->str == "mlstm") {
        s.mixer = MIX_MLSTM;
        s.kv_heads = s.heads;
        if (s.dim > 1024) { *err = "config: " + where + "mixer.dim above 1024"; return false; }
        if (jnum(mx, "gate_cap", &d) && d > 0) s.gate_cap = static_cast<float>(d);
      } else {
        *err = "config: unknown mixer \"" + ty->str + "\"";
        return false;
      }
      const JVal* mlp = L.get("mlp");
      if (mlp && mlp->type == JVal::Obj) {
        const JVal* kind = mlp->get("kind");
        if (!kind || kind->type != JVal::Str) { *err = "config: " + where + "mlp.kind"; return false; }
        if (kind->str == "dense") {
          s.mlp = MLP_DENSE;
          if (!whole(mlp, "ff", 1, &s.ff, where + "mlp.")) return false;
        } else if (kind->str == "moe") {
          s.mlp = MLP_MOE;
          const JVal* ex = mlp->get("expert");
          const JVal* ro = mlp->get("router");
          if (!whole(ex, "ff", 1, &s.ff, where + "mlp.expert.") || !whole(ro, "experts", 1, &s.experts, where + "mlp.router.") ||
              !whole(ro, "top", 1, &s.top, where + "mlp.router.")) return false;
          if (s.top > s.experts) { *err = "config: " + where + "mlp.router.top above experts"; return false; }
          const JVal* sh = mlp->get("shared");
          if (sh && sh->type == JVal::Obj) {
            s.shared = true;
            if (!whole(sh, "ff", 1, &s.sff, where + "mlp.shared.")) return false;
          }
        } else {
          *err = "config: " + where + "mlp.kind \"" + kind->str + "\"";
          return false;
        }
      }
      layout(s);
      spec.push_back(s);
    }
    return true;
  }

  static int up8(int v) { return (v + 7) / 8 * 8; }
  void layout(LayerSpec& s) {
    int at = 0;
    auto block = [&](int* off, int n) { *off = at; at = up8(at + n); };   // every block starts 16-byte aligned
    block(&s.off_q, s.heads * s.dim);
    block(&s.off_k, s.kv_heads * s.dim);
    block(&s.off_v, s.kv_heads * s.vdim);
    block(&s.off_g, s.mixer == MIX_ATTENTION ? s.heads : s.heads * s.vdim);   // one gate logit per head / per output column
    s.n_in = at;
    s.k_out = s.heads * s.vdim;
    s.n_sh = s.shared ? up8(2 * s.sff) : 0;
  }

  template <typename P>
  int dalloc(P** p, size_t bytes) {
    void* q = nullptr;
    if (cudaMalloc(&q, std::max<size_t>(bytes, 16)) != cudaSuccess) { set_error("Mulenex: device allocation of %zu bytes failed", bytes); return -3; }
    cudaMemsetAsync(q, 0, std::max<size_t>(bytes, 16), env.stream);
    allocs.push_back(q);
    *p = static_cast<P*>(q);
    return 0;
  }

  int init(const ModelEnv& e) override {
    env = e;
    const size_t es = dtype_bytes(dt);
    wts.resize(spec.size());
    int max_in = 8, max_kout = 8, max_qn = 1, max_o = 1, max_h = 1, max_e = 1, max_top = 1, max_eff = 1, max_ff = 1, max_nsh = 8, max_sff = 1;
    bool any_moe = false, any_shared = false, any_dense = false, any_mlstm = false;
    for (auto& s : spec) {
      max_in = std::max(max_in, s.n_in);
      max_kout = std::max(max_kout, s.k_out);
      if (s.mixer == MIX_ATTENTION) max_qn = std::max(max_qn, s.heads * s.dim);
      else { any_mlstm = true; max_o = std::max(max_o, s.heads * s.vdim); max_h = std::max(max_h, s.heads); }
      if (s.v_first) vfirst_ld = up8(s.kv_heads * s.vdim);
      if (s.mlp == MLP_DENSE) { any_dense = true; max_ff = std::max(max_ff, s.ff); }
      if (s.mlp == MLP_MOE) {
        any_moe = true;
        max_e = std::max(max_e, s.experts + 1); max_top = std::max(max_top, s.top); max_eff = std::max(max_eff, s.ff);
        if (s.shared) { any_shared = true; max_nsh = std::max(max_nsh, s.n_sh); max_sff = std::max(max_sff, s.sff); }
      }
    }
    int rc = 0;
    auto mat = [&](void** p, size_t rows, size_t cols) { return dalloc(p, rows * cols * es); };
    auto vec = [&](float** p, size_t n) { return dalloc(p, n * sizeof(float)); };
    rc |= mat(&embed, V, W) | mat(&head, V, W) | vec(&fin_w, W) | dalloc(&pos_freq, static_cast<size_t>((W + 1) / 2) * sizeof(float2));
    if (!rc && sinusoid_freq_table(pos_freq, W, 10000.0, e.stream)) rc = -2;
    for (size_t i = 0; i < spec.size() && !rc; ++i) {
      const LayerSpec& s = spec[i];
      LayerWeights& w = wts[i];
      rc |= mat(&w.w_in, s.n_in, W) | mat(&w.w_out, W, s.k_out) | vec(&w.norm1, W) | vec(&w.norm1b, W);
      if (s.mixer == MIX_ATTENTION) {
        rc |= vec(&w.q_norm, s.dim) | vec(&w.k_norm, s.dim);
        rc |= dalloc(&w.cache, static_cast<size_t>(e.num_blocks) * e.page * s.kv_heads * (s.dim + s.vdim) * es);
      } else {
        rc |= mat(&w.w_gates, 2 * s.heads, W) | vec(&w.b_gates, 2 * s.heads) | vec(&w.h_norm, static_cast<size_t>(s.heads) * s.vdim);
        rc |= dalloc(&w.state, static_cast<size_t>(e.num_slots) * s.heads * s.dim * s.vdim * sizeof(float));
        rc |= dalloc(&w.nstate, static_cast<size_t>(e.num_slots) * s.heads * s.dim * sizeof(float));
        rc |= dalloc(&w.mstate, static_cast<size_t>(e.num_slots) * s.heads * sizeof(float));
      }
      if (s.mlp != MLP_NONE) rc |= vec(&w.norm2, W) | vec(&w.norm2b, W);
      if (s.mlp == MLP_DENSE) rc |= mat(&w.up, s.ff, W) | mat(&w.down, W, s.ff) | vec(&w.up_b, s.ff) | vec(&w.down_b, W);
      if (s.mlp == MLP_MOE) {
        const int nr = s.experts + (s.shared ? 1 : 0);
        rc |= mat(&w.router, nr, W) | vec(&w.router_b, nr) | mat(&w.e_gu, static_cast<size_t>(s.experts) * 2 * s.ff, W) |
              mat(&w.e_down, static_cast<size_t>(s.experts) * W, s.ff);
        if (s.shared) rc |= mat(&w.sh_in, s.n_sh, W) | mat(&w.sh_down, W, s.sff);
      }
    }
    if (rc) return rc;
    const size_t T = e.Tcap;
    row_cap = static_cast<int>(std::min<size_t>(T, 256));
    rc |= dalloc(&x, T * W * sizeof(float)) | mat(&h, T, W) | mat(&inb, T, max_in) | mat(&ycat, T, max_kout) | mat(&ao, T, W) | mat(&hrow, row_cap, W);
    rc |= dalloc(&qn, T * max_qn * sizeof(float)) | dalloc(&logits, static_cast<size_t>(row_cap) * V * sizeof(float));
    if (vfirst_ld) rc |= mat(&vfirst, T, vfirst_ld);
    if (any_mlstm)
      rc |= dalloc(&o32, T * max_o * sizeof(float)) | dalloc(&gpre, T * 2 * max_h * sizeof(float)) | dalloc(&gkeep, T * max_h * sizeof(float)) |
            dalloc(&gtake, T * max_h * sizeof(float)) | dalloc(&gfloor, T * max_h * sizeof(float)) | dalloc(&gnq, T * max_h * sizeof(float));
    if (any_dense) rc |= mat(&ffh, T, max_ff);
    if (any_dense || any_moe) rc |= mat(&fo, T, W);
    if (any_moe) {
      moe_cap = static_cast<int>((T * max_top + 63) / 64 * 64) + max_e * 64;
      rc |= dalloc(&scores, T * max_e * sizeof(float)) | dalloc(&topw, T * max_top * sizeof(float)) | dalloc(&topi, T * max_top * sizeof(int)) |
            dalloc(&sorted_rows, static_cast<size_t>(moe_cap) * sizeof(int)) | dalloc(&tile_group, static_cast<size_t>(moe_cap / 64) * sizeof(int)) |
            dalloc(&pair_pos, T * max_top * sizeof(int)) | mat(&egu, moe_cap, 2 * static_cast<size_t>(max_eff)) | mat(&eact, moe_cap, max_eff) |
            dalloc(&edown, static_cast<size_t>(moe_cap) * W * sizeof(float)) | dalloc(&iota, static_cast<size_t>(64) * sizeof(int));
      if (!rc) {
        int hi[64];
        for (int i = 0; i < 64; ++i) hi[i] = i;
        if (cudaMemcpyAsync(iota, hi, sizeof(hi), cudaMemcpyHostToDevice, e.stream) != cudaSuccess || cudaStreamSynchronize(e.stream) != cudaSuccess) rc = -2;
      }
      if (any_shared) rc |= mat(&sh, T, max_nsh) | mat(&shact, T, max_sff) | mat(&sdown, T, W);
    }
    if (rc) return rc;
    register_tensors();
    rc = setup_tc();
    if (rc) return rc;
    return cudaStreamSynchronize(e.stream) == cudaSuccess ? 0 : -2;
  }

  // The projections of a bf16 model run on the tcgen05 pair GEMM (gemm2_tcgen05.cu) where their shapes allow it (K % 8 == 0):
  // input and output projection, the dense feed-forward, the shared expert, and every expert for steps large enough to sort
  // rows per expert.  B200_MX_TC=0 keeps every projection on linear.cu (A/B knob); fp32 models always do.
  int setup_tc() {
    const char* ev = getenv("B200_MX_TC");
    use_tc = dt == DT_BF16 && !(ev && atoi(ev) == 0) && W % 8 == 0 && gemm_variant() == 2;
    if (!use_tc) return 0;
    int maxN = W;
    for (auto& s : spec) maxN = std::max(std::max(maxN, s.n_in), std::max(s.n_sh, std::max(2 * s.ff, s.ff)));
    const size_t ws_bytes = std::max(gemm_workspace_bytes(env.sms), gemm_deferred_ws_bytes(env.sms));
    if (dalloc(&gemm_ws, ws_bytes)) return -3;
    const size_t n_counters = 2ull * (maxN / 128 + 2) * (env.Tcap / 32 + 2);
    if (dalloc(&gemm_counters, n_counters * sizeof(int))) return -3;
    const int bns[kGemmNumBlockN] = {32, 64, 128, 256, 512};
    for (int i = 0; i < kGemmNumBlockN; ++i)
      if (gemm_make_x_map(&xm_h[i], h, env.Tcap, W, W, bns[i])) { use_tc = false; return 0; }
    auto plan = [&](GemmPlan* p, const void* Wm, int N, int K) {
      if (K % 8 || gemm_plan_init(p, Wm, N, K, K, gemm_ws, gemm_counters, env.sms)) return false;
      p->ws_bytes = ws_bytes;
      return true;
    };
    auto maps = [&](CUtensorMap* xm, const void* X, int K) {
      for (int j = 0; j < kGemmNumBlockN; ++j)
        if (gemm_make_x_map(&xm[j], X, env.Tcap, K, K, bns[j])) return false;
      return true;
    };
    bool any_expert_tc = false;
    for (size_t i = 0; i < spec.size(); ++i) {
      const LayerSpec& s = spec[i];
      LayerWeights& w = wts[i];
      w.tc_in = plan(&w.p_in, w.w_in, s.n_in, W);
      w.tc_out = plan(&w.p_out, w.w_out, W, s.k_out);
      if (w.tc_out && !maps(w.xm_out, ycat, s.k_out)) { gemm_plan_destroy(&w.p_out); w.tc_out = false; }
      if (s.mlp == MLP_DENSE) {
        w.tc_up = plan(&w.p_up, w.up, s.ff, W);
        w.tc_down = plan(&w.p_down, w.down, W, s.ff);
        if (w.tc_down && !maps(w.xm_ffh, ffh, s.ff)) { gemm_plan_destroy(&w.p_down); w.tc_down = false; }
      }
      if (s.mlp == MLP_MOE && s.shared) {
        w.tc_shin = plan(&w.p_shin, w.sh_in, s.n_sh, W);
        w.tc_shdown = plan(&w.p_shdown, w.sh_down, W, s.sff);
        if (w.tc_shdown && !maps(w.xm_shact, shact, s.sff)) { gemm_plan_destroy(&w.p_shdown); w.tc_shdown = false; }
      }
      if (s.mlp == MLP_MOE && s.ff % 8 == 0) {
        w.p_egu.resize(s.experts);
        w.p_edown.resize(s.experts);
        int made_u = 0, made_d = 0;
        bool ok = true;
        for (int e = 0; e < s.experts && ok; ++e) {
          ok = plan(&w.p_egu[e], static_cast<bf16*>(w.e_gu) + static_cast<size_t>(e) * 2 * s.ff * W, 2 * s.ff, W);
          if (ok) ++made_u;
          ok = ok && plan(&w.p_edown[e], static_cast<bf16*>(w.e_down) + static_cast<size_t>(e) * W * s.ff, W, s.ff);
          if (ok) ++made_d;
        }
        if (!ok) {
          for (int e = 0; e < made_u; ++e) gemm_plan_destroy(&w.p_egu[e]);
          for (int e = 0; e < made_d; ++e) gemm_plan_destroy(&w.p_edown[e]);
          w.p_egu.clear(); w.p_edown.clear();
        } else any_expert_tc = true;
      }
    }
    if (any_expert_tc) {
      int max_e = 1;
      for (auto& s : spec) max_e = std::max(max_e, s.experts);
      if (dalloc(&hsorted, static_cast<size_t>(moe_cap) * W * 2) || dalloc(&edown16, static_cast<size_t>(moe_cap) * W * 2) ||
          dalloc(&expert_rows, static_cast<size_t>(max_e) * 2 * sizeof(int))) return -3;
      if (cudaMallocHost(&expert_rows_host, static_cast<size_t>(max_e) * 2 * sizeof(int)) != cudaSuccess) return -3;
    }
    return 0;
  }

  void reg(const std::string& name, void* p, size_t bytes) { tensors[name] = {p, bytes}; }
  void register_tensors() {
    const size_t es = dtype_bytes(dt);
    reg("embed", embed, static_cast<size_t>(V) * W * es);
    reg("head", head, static_cast<size_t>(V) * W * es);
    for (size_t i = 0; i < spec.size(); ++i) {
      const std::string p = "l" + std::to_string(i) + ".";
      reg(p + "w_in", wts[i].w_in, static_cast<size_t>(spec[i].n_in) * W * es);
      reg(p + "w_out", wts[i].w_out, static_cast<size_t>(W) * spec[i].k_out * es);
    }
  }

  // ------------------------------------------------------------ weights
  // host fp32 [rows, cols] -> device rows [row0, row0 + rows) x columns [col0, col0 + cols) of a matrix with leading dimension ld
  int put(void* dst, size_t ld, size_t row0, size_t col0, const std::vector<float>& src, size_t rows, size_t cols) {
    const size_t es = dtype_bytes(dt);
    std::vector<uint8_t> tmp(rows * cols * es);
    if (dt == DT_F32) memcpy(tmp.data(), src.data(), tmp.size());
    else {
      bf16* o = reinterpret_cast<bf16*>(tmp.data());
      for (size_t i = 0; i < rows * cols; ++i) o[i] = __float2bfloat16_rn(src[i]);
    }
    uint8_t* d = static_cast<uint8_t*>(dst) + (row0 * ld + col0) * es;
    return cudaMemcpy2D(d, ld * es, tmp.data(), cols * es, cols * es, rows, cudaMemcpyHostToDevice) == cudaSuccess ? 0 : -2;
  }
  int putf(float* dst, const std::vector<float>& src, float offset = 0.f) {
    std::vector<float> t(src);
    for (auto& v : t) v += offset;
    return cudaMemcpy(dst, t.data(), t.size() * sizeof(float), cudaMemcpyHostToDevice) == cudaSuccess ? 0 : -2;
  }

  int load(const CheckpointReader& ck, std::string* err) override {
    std::vector<float> v;
    std::vector<int64_t> sh;
    auto get = [&](const std::string& name, int64_t rows, int64_t cols) {
      if (!ck.read_f32(name, &v, &sh, err)) return false;
      int64_t n = 1;
      for (auto d : sh) n *= d;
      const int64_t r = sh.size() == 2 ? sh[0] : 1, c = sh.size() == 2 ? sh[1] : n;
      if (r != rows || c != cols) {
        *err = name + ": shape [" + std::to_string(r) + "," + std::to_string(c) + "] does not fit the config";
        return false;
      }
      return true;
    };
    int rc = 0;
#define MAT(name, dst, ld, row0, col0, rows, cols) do { if (!get(name, rows, cols)) return -4; rc |= put(dst, ld, row0, col0, v, rows, cols); } while (0)
#define VEC(name, dst, n) do { if (!get(name, 1, n)) return -4; rc |= putf(dst, v); } while (0)
#define NORM(name, dst, n) do { if (!get(name, 1, n)) return -4; rc |= putf(dst, v, 1.0f); } while (0)   // stored as the offset from one
    MAT("embed", embed, W, 0, 0, V, W);
    MAT("head", head, W, 0, 0, V, W);
    NORM("final.norm", fin_w, W);
    for (size_t i = 0; i < spec.size(); ++i) {
      const LayerSpec& s = spec[i];
      LayerWeights& w = wts[i];
      const std::string p = "l" + std::to_string(i) + ".", m = p + "mix.", f = p + "mlp.";
      NORM(p + "norm1", w.norm1, W);
      NORM(p + "norm1b", w.norm1b, W);
      MAT(m + "q", w.w_in, W, s.off_q, 0, s.heads * s.dim, W);
      MAT(m + "k", w.w_in, W, s.off_k, 0, s.kv_heads * s.dim, W);
      MAT(m + "v", w.w_in, W, s.off_v, 0, s.kv_heads * s.vdim, W);
      MAT(m + "o", w.w_out, s.k_out, 0, 0, W, s.k_out);
      if (s.mixer == MIX_ATTENTION) {
        MAT(m + "g", w.w_in, W, s.off_g, 0, s.heads, W);
        VEC(m + "q.norm", w.q_norm, s.dim);
        VEC(m + "k.norm", w.k_norm, s.dim);
        if (s.v_mix && !s.v_first) {
          if (!get(m + "vmix", 1, 1)) return -4;
          w.v_lambda = v[0];
        }
      } else {
        MAT(m + "g", w.w_in, W, s.off_g, 0, s.heads * s.vdim, W);
        MAT(m + "i", w.w_gates, W, 0, 0, s.heads, W);
        MAT(m + "f", w.w_gates, W, s.heads, 0, s.heads, W);
        std::vector<float> b;
        if (!get(m + "i.b", 1, s.heads)) return -4;
        b = v;
        if (!get(m + "f.b", 1, s.heads)) return -4;
        b.insert(b.end(), v.begin(), v.end());
        rc |= putf(w.b_gates, b);
        VEC(m + "norm", w.h_norm, s.heads * s.vdim);
      }
      if (s.mlp == MLP_NONE) continue;
      NORM(p + "norm2", w.norm2, W);
      NORM(p + "norm2b", w.norm2b, W);
      if (s.mlp == MLP_DENSE) {
        MAT(f + "up", w.up, W, 0, 0, s.ff, W);
        MAT(f + "down", w.down, s.ff, 0, 0, W, s.ff);
        VEC(f + "up.b", w.up_b, s.ff);
        VEC(f + "down.b", w.down_b, W);
        continue;
      }
      MAT(f + "router", w.router, W, 0, 0, s.experts, W);
      if (!get(f + "router.b", 1, s.experts)) return -4;
      {
        std::vector<float> b(v);
        if (s.shared) b.push_back(0.f);
        rc |= putf(w.router_b, b);
      }
      for (int e = 0; e < s.experts; ++e) {
        const std::string ep = f + "e" + std::to_string(e) + ".";
        MAT(ep + "gate", w.e_gu, W, static_cast<size_t>(e) * 2 * s.ff, 0, s.ff, W);
        MAT(ep + "up", w.e_gu, W, static_cast<size_t>(e) * 2 * s.ff + s.ff, 0, s.ff, W);
        MAT(ep + "down", w.e_down, s.ff, static_cast<size_t>(e) * W, 0, W, s.ff);
      }
      if (s.shared) {
        MAT(f + "shared.gate", w.sh_in, W, 0, 0, s.sff, W);
        MAT(f + "shared.up", w.sh_in, W, s.sff, 0, s.sff, W);
        MAT(f + "shared.sg", w.router, W, s.experts, 0, 1, W);
        MAT(f + "shared.down", w.sh_down, s.sff, 0, 0, W, s.sff);
      }
    }
#undef MAT
#undef VEC
#undef NORM
    if (rc) { *err = "copying weights to the device failed"; return -2; }
    return 0;
  }

  // Seeded random weights of a plausible scale (benchmarks: there is no checkpoint of a real size).
  int randomize(uint64_t seed) override {
    cudaStream_t st = env.stream;
    int rc = 0;
    uint64_t k = seed * 1000003ull + 41;
    auto M = [&](void* p, size_t n, float sc) { if (p) rc |= fill_uniform(p, dt, n, ++k, sc, 0.f, st); };
    auto F = [&](float* p, size_t n, float sc, float off) { if (p) rc |= fill_uniform(p, DT_F32, n, ++k, sc, off, st); };
    const float sw = 1.7f / sqrtf(static_cast<float>(W));
    M(embed, static_cast<size_t>(V) * W, 1.0f);
    M(head, static_cast<size_t>(V) * W, sw);
    F(fin_w, W, 0.1f, 1.f);
    for (size_t i = 0; i < spec.size(); ++i) {
      const LayerSpec& s = spec[i];
      LayerWeights& w = wts[i];
      M(w.w_in, static_cast<size_t>(s.n_in) * W, sw);
      M(w.w_out, static_cast<size_t>(W) * s.k_out, 1.7f / sqrtf(static_cast<float>(s.k_out)));
      F(w.norm1, W, 0.1f, 1.f); F(w.norm1b, W, 0.1f, 1.f); F(w.norm2, W, 0.1f, 1.f); F(w.norm2b, W, 0.1f, 1.f);
      F(w.q_norm, s.dim, 0.1f, 1.f); F(w.k_norm, s.dim, 0.1f, 1.f);
      w.v_lambda = s.v_mix && !s.v_first ? 0.3f : 0.f;
      M(w.w_gates, static_cast<size_t>(2) * s.heads * W, sw);
      F(w.b_gates, 2 * s.heads, 1.f, 1.f);
      F(w.h_norm, static_cast<size_t>(s.heads) * s.vdim, 0.1f, 1.f);
      if (s.mlp == MLP_DENSE) {
        M(w.up, static_cast<size_t>(s.ff) * W, sw); M(w.down, static_cast<size_t>(W) * s.ff, 1.7f / sqrtf(static_cast<float>(s.ff)));
        F(w.up_b, s.ff, 0.1f, 0.f); F(w.down_b, W, 0.1f, 0.f);
      }
      if (s.mlp == MLP_MOE) {
        M(w.router, static_cast<size_t>(s.experts + (s.shared ? 1 : 0)) * W, sw);
        F(w.router_b, s.experts, 0.1f, 0.f);
        M(w.e_gu, static_cast<size_t>(s.experts) * 2 * s.ff * W, sw);
        M(w.e_down, static_cast<size_t>(s.experts) * W * s.ff, 1.7f / sqrtf(static_cast<float>(s.ff)));
        if (s.shared) { M(w.sh_in, static_cast<size_t>(s.n_sh) * W, sw); M(w.sh_down, static_cast<size_t>(W) * s.sff, 1.7f / sqrtf(static_cast<float>(s.sff))); }
      }
    }
    if (rc) return -2;
    return cudaStreamSynchronize(st) == cudaSuccess ? 0 : -2;
  }

  // ------------------------------------------------------------ forward
  int project(const GemmPlan& plan, bool tc, const CUtensorMap* xm, const void* X, const void* Wm, void* Y, int T, int N, int K,
              const float* bias = nullptr, int act = LIN_NONE) {
    if (tc) {
      const int bn = gemm_block_n_for(T);
      int rc = gemm_run(plan, xm[gemm_block_n_index(bn)], bn, Y, N, T, env.stream);
      if (!rc && (bias || act != LIN_NONE)) rc = bias_act(Y, N, bias, act, dt, T, N, env.stream);
      return rc;
    }
    LinearArgs a = linear_args(X, dt, Wm, dt, Y, dt, T, N, K);
    a.bias = bias; a.act = act;
    return linear(a, env.stream);
  }

  // per-kernel device time (b200_engine_kernel_times): with profiling on, every launch is bracketed by events and waited for
  cudaEvent_t pe0 = nullptr, pe1 = nullptr;
  void prof_start() {
    if (!profile_kernels) return;
    if (!pe0) { cudaEventCreate(&pe0); cudaEventCreate(&pe1); }
    cudaEventRecord(pe0, env.stream);
  }
  void prof_stop(const char* name) {
    if (!profile_kernels) return;
    cudaEventRecord(pe1, env.stream);
    cudaEventSynchronize(pe1);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, pe0, pe1);
    auto& t = kernel_times[name];
    t.first += ms * 1000.0;
    t.second += 1;
  }
#define KRN(name, call) do { prof_start(); const int r_ = (call); if (r_ && !rc) { failed_kernel = name; failed_rc = r_; } rc |= r_; prof_stop(name); ++nl; } while (0)
  const char* failed_kernel = "";
  int failed_rc = 0;

  // the output of the last sublayer, still to be normed and added by the next boundary kernel
  struct Pending {
    const void* y = nullptr;
    const float* bias = nullptr;
    const float* post_w = nullptr;
  };
  SandwichArgs boundary(const Pending& p, const float* pre_w, void* out, DType to, const int* row_index, int rows) {
    SandwichArgs a;
    a.x = x; a.y = p.y; a.ty = dt; a.y_bias = p.bias; a.post_w = p.post_w; a.pre_w = pre_w; a.eps = eps;
    a.h = out; a.th = to; a.row_index = row_index; a.rows = rows; a.W = W;
    return a;
  }

  int attention(const LayerSpec& s, const LayerWeights& w, const StepBatch& b, int64_t& nl) {
    cudaStream_t st = env.stream;
    const size_t es = dtype_bytes(dt);
    auto col = [&](void* base, size_t off) { return static_cast<void*>(static_cast<uint8_t*>(base) + off * es); };
    int rc = 0;
    QkPrepArgs qp;
    qp.q = col(inb, s.off_q); qp.k = col(inb, s.off_k); qp.v = col(inb, s.off_v); qp.ld = s.n_in; qp.t = dt;
    qp.rope = nullptr; qp.rot_dims = 0; qp.unit_norm = true; qp.eps = eps;
    qp.positions = b.pos; qp.slots = b.slots; qp.qn = qn; qp.cache = w.cache;
    qp.T = b.T; qp.heads = s.heads; qp.kv_heads = s.kv_heads; qp.dim = s.dim; qp.vdim = s.vdim;
    qp.q_norm_w = w.q_norm; qp.k_norm_w = w.k_norm; qp.q_gain_coef = s.qt_coef; qp.q_gain_every = s.qt_every;
    if (s.v_first) { qp.v_raw_out = vfirst; qp.ld_raw = vfirst_ld; }
    else if (s.v_mix) { qp.v_blend = vfirst; qp.ld_blend = vfirst_ld; qp.v_lambda = w.v_lambda; }
    KRN("qk_prep", qk_rope_norm_cache(qp, st));
    WindowAttnArgs wa;
    wa.qn = qn; wa.cache = w.cache; wa.t = dt; wa.positions = b.pos; wa.seq_of_tok = b.seq_of_tok; wa.block_tables = b.btab;
    wa.max_blocks = b.max_blocks; wa.page = env.page;
    wa.gate = col(inb, s.off_g); wa.ldg = s.n_in; wa.gate_per_head = true; wa.out_scale = 1.f; wa.y = ycat; wa.ldy = s.k_out;
    wa.T = b.T; wa.heads = s.heads; wa.kv_heads = s.kv_heads; wa.dim = s.dim; wa.vdim = s.vdim;
    wa.window = 1 << 30; wa.keep_first = 0; wa.scale = s.scale; wa.softcap = s.softcap;
    wa.seqs = b.seqs; wa.nseq = b.nseq; wa.max_ctx = b.max_ctx;
    KRN("attention", window_attention(wa, st));
    return rc;
  }

  int mlstm(const LayerSpec& s, const LayerWeights& w, const StepBatch& b, int64_t& nl) {
    cudaStream_t st = env.stream;
    const size_t es = dtype_bytes(dt);
    auto col = [&](void* base, size_t off) { return static_cast<void*>(static_cast<uint8_t*>(base) + off * es); };
    int rc = 0;
    // gate pre-activations in fp32 straight from the accumulator, bias included
    LinearArgs ga = linear_args(h, dt, w.w_gates, dt, gpre, DT_F32, b.T, 2 * s.heads, W);
    ga.bias = w.b_gates;
    KRN("mlstm_gate_proj", linear(ga, st));
    MlstmGateArgs mg;
    mg.pre = gpre; mg.ld = 2 * s.heads; mg.cap = s.gate_cap; mg.keep = gkeep; mg.take = gtake; mg.floor = gfloor;
    mg.mstate = w.mstate; mg.seqs = b.seqs; mg.nseq = b.nseq; mg.heads = s.heads;
    KRN("mlstm_gates", mlstm_gates(mg, st));
    GlaArgs g;
    g.qkv = inb; g.t = dt; g.ld = s.n_in; g.q_off = s.off_q; g.k_off = s.off_k; g.v_off = s.off_v;
    g.z = nullptr; g.z_bias = nullptr; g.inv_tau = 1.f; g.q_scale = 1.0f / sqrtf(static_cast<float>(s.dim)); g.T = b.T;
    g.states = w.state; g.seqs = b.seqs; g.nseq = b.nseq;
    g.heads = s.heads; g.dim = s.dim; g.vdim = s.vdim; g.o = o32;
    g.tok_decay = gkeep; g.tok_kscale = gtake; g.nstate = w.nstate; g.nq = gnq;
    KRN("mlstm_scan", gla_scan(g, st));
    OutGateArgs og;
    og.o = o32; og.g = col(inb, s.off_g); og.ldg = s.n_in; og.w = w.h_norm; og.eps = eps;
    og.y = ycat; og.ldy = s.k_out; og.t = dt; og.T = b.T; og.heads = s.heads; og.vdim = s.vdim;
    og.joint = false; og.gate_act = GATE_SIGMOID; og.out_scale = 1.f;
    og.w_full = true; og.den_nq = gnq; og.den_floor = gfloor; og.den_eps = 1e-6f;
    KRN("mlstm_out_gate", recurrent_out_gate(og, st));
    return rc;
  }

  int dense(const LayerSpec& s, const LayerWeights& w, int T, int64_t& nl) {
    int rc = 0;
    KRN("ff_up", project(w.p_up, w.tc_up, xm_h, h, w.up, ffh, T, s.ff, W, w.up_b, LIN_RELU2));
    KRN("ff_down", project(w.p_down, w.tc_down, w.xm_ffh, ffh, w.down, fo, T, W, s.ff));   // its bias joins in the boundary kernel
    return rc;
  }

  int moe(const LayerSpec& s, const LayerWeights& w, int T, int64_t& nl) {
    cudaStream_t st = env.stream;
    int rc = 0;
    const int nr = s.experts + (s.shared ? 1 : 0);   // router logits and, behind them, the shared expert's gate logit
    LinearArgs ra = linear_args(h, dt, w.router, dt, scores, DT_F32, T, nr, W);
    ra.bias = w.router_b;
    KRN("moe_router", linear(ra, st));
    KRN("moe_route", moe_route(scores, topi, topw, T, s.experts, 1, 1, s.top, st, MOE_TOP_SOFTMAX, nr));
    const void* shared_out = nullptr;
    const float* shared_gate = nullptr;
    if (s.shared) {
      KRN("shared_in", project(w.p_shin, w.tc_shin, xm_h, h, w.sh_in, sh, T, s.n_sh, W));
      KRN("glu", glu_clamped(sh, s.n_sh, shact, s.sff, dt, T, s.sff, INFINITY, 1.f, st, 0.f));
      KRN("shared_down", project(w.p_shdown, w.tc_shdown, w.xm_shact, shact, w.sh_down, sdown, T, W, s.sff));
      shared_out = sdown;
      shared_gate = scores + s.experts;
    }
    const long long gu_stride = 2ll * s.ff * W, down_stride = static_cast<long long>(W) * s.ff;
    static const int moe_tc_min = [] { const char* e = getenv("B200_MX_MOE_TC_MIN_T"); return e ? atoi(e) : 256; }();   // A/B knob
    const bool per_expert = !w.p_egu.empty() && T >= moe_tc_min;
    if (T * s.top <= 64) {
      // decode-sized steps: one weight-streaming pass per chosen (token, expert) pair, rows in pair order
      LinearArgs up = linear_args(h, dt, w.e_gu, dt, egu, dt, T * s.top, 2 * s.ff, W);
      up.wbs = gu_stride;
      const PickedRows pu = {T * s.top, nullptr, s.top, iota, topi};
      KRN("moe_up", linear_picked_rows(up, pu, st));
      KRN("glu", glu_clamped(egu, 2 * s.ff, eact, s.ff, dt, T * s.top, s.ff, INFINITY, 1.f, st, 0.f));
      LinearArgs dn = linear_args(eact, dt, w.e_down, dt, edown, DT_F32, T * s.top, W, s.ff);
      dn.wbs = down_stride;
      const PickedRows pd = {T * s.top, iota, 1, iota, topi};
      KRN("moe_down", linear_picked_rows(dn, pd, st));
      // pair k of token t is row t * top + k: the combine walks them through an identity table
      KRN("moe_combine", moe_combine_add(edown, DT_F32, iota, topw, shared_out, shared_gate, nr, fo, dt, T, s.top, W, st));
      return rc;
    }
    const int cap = (T * s.top + 63) / 64 * 64 + s.experts * 64;
    KRN("moe_align", moe_align(topi, T, s.top, s.experts, sorted_rows, tile_group, pair_pos, cap, st, per_expert ? expert_rows : nullptr));
    if (per_expert) {
      // Large steps: every expert's rows are one tcgen05 GEMM.  The row counts come back to the host (one small copy and a
      // wait per layer, paid only by steps of hundreds of tokens); the inputs are gathered into sorted order.
      KRN("moe_gather", moe_gather_bf16(h, sorted_rows, hsorted, cap, W, st));
      if (cudaMemcpyAsync(expert_rows_host, expert_rows, static_cast<size_t>(s.experts) * 2 * sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
          cudaStreamSynchronize(st) != cudaSuccess) rc = -2;
      prof_start();
      for (int e = 0; e < s.experts && !rc; ++e) {
        const int start = expert_rows_host[2 * e], cnt = expert_rows_host[2 * e + 1];
        if (cnt <= 0) continue;
        const int bn = gemm_block_n_for(cnt);
        CUtensorMap tm;
        if (gemm_make_x_map(&tm, static_cast<bf16*>(hsorted) + static_cast<size_t>(start) * W, cnt, W, W, bn)) { rc = -2; break; }
        rc |= gemm_run(w.p_egu[e], tm, bn, static_cast<bf16*>(egu) + static_cast<size_t>(start) * 2 * s.ff, 2 * s.ff, cnt, st);
        ++nl;
      }
      prof_stop("moe_up");
      KRN("glu", glu_clamped(egu, 2 * s.ff, eact, s.ff, dt, cap, s.ff, INFINITY, 1.f, st, 0.f));
      prof_start();
      for (int e = 0; e < s.experts && !rc; ++e) {
        const int start = expert_rows_host[2 * e], cnt = expert_rows_host[2 * e + 1];
        if (cnt <= 0) continue;
        const int bn = gemm_block_n_for(cnt);
        CUtensorMap tm;
        if (gemm_make_x_map(&tm, static_cast<bf16*>(eact) + static_cast<size_t>(start) * s.ff, cnt, s.ff, s.ff, bn)) { rc = -2; break; }
        rc |= gemm_run(w.p_edown[e], tm, bn, static_cast<bf16*>(edown16) + static_cast<size_t>(start) * W, W, cnt, st);
        ++nl;
      }
      prof_stop("moe_down");
      KRN("moe_combine", moe_combine_add(edown16, DT_BF16, pair_pos, topw, shared_out, shared_gate, nr, fo, dt, T, s.top, W, st));
      return rc;
    }
    LinearArgs up = linear_args(h, dt, w.e_gu, dt, egu, dt, cap, 2 * s.ff, W);
    up.x_rows = sorted_rows; up.tile_group = tile_group; up.wbs = gu_stride;
    KRN("moe_up", linear(up, st));
    KRN("glu", glu_clamped(egu, 2 * s.ff, eact, s.ff, dt, cap, s.ff, INFINITY, 1.f, st, 0.f));
    LinearArgs dn = linear_args(eact, dt, w.e_down, dt, edown, DT_F32, cap, W, s.ff);
    dn.tile_group = tile_group; dn.wbs = down_stride;
    KRN("moe_down", linear(dn, st));
    KRN("moe_combine", moe_combine_add(edown, DT_F32, pair_pos, topw, shared_out, shared_gate, nr, fo, dt, T, s.top, W, st));
    return rc;
  }

  int forward(const StepBatch& b, int* sampled, float* host_logits, int64_t* launches) override {
    cudaStream_t st = env.stream;
    const int T = b.T;
    int rc = 0;
    int64_t nl = 0;
    KRN("embed", embed_sinusoid(embed, dt, b.ids, b.pos, pos_freq, x, T, W, V, st));
    Pending pend;
    for (size_t li = 0; li < spec.size() && !rc; ++li) {
      const LayerSpec& s = spec[li];
      const LayerWeights& w = wts[li];
      KRN("residual_norm", sandwich_step(boundary(pend, w.norm1, h, dt, nullptr, T), st));
      KRN("proj_in", project(w.p_in, w.tc_in, xm_h, h, w.w_in, inb, T, s.n_in, W));
      rc |= s.mixer == MIX_ATTENTION ? attention(s, w, b, nl) : mlstm(s, w, b, nl);
      KRN("proj_out", project(w.p_out, w.tc_out, w.xm_out, ycat, w.w_out, ao, T, W, s.k_out));
      pend = Pending();
      pend.y = ao; pend.post_w = w.norm1b;
      if (s.mlp != MLP_NONE) {
        KRN("residual_norm", sandwich_step(boundary(pend, w.norm2, h, dt, nullptr, T), st));
        rc |= s.mlp == MLP_DENSE ? dense(s, w, T, nl) : moe(s, w, T, nl);
        pend = Pending();
        pend.y = fo; pend.post_w = w.norm2b; pend.bias = s.mlp == MLP_DENSE ? w.down_b : nullptr;
      }
      if (residual_sink && !rc) {
        // debug: apply the write-back now and read the residual
        KRN("residual_norm", sandwich_step(boundary(pend, nullptr, nullptr, dt, nullptr, T), st));
        pend = Pending();
        const size_t at = residual_sink->size();
        residual_sink->resize(at + static_cast<size_t>(T) * W);
        if (rc || cudaMemcpyAsync(residual_sink->data() + at, x, static_cast<size_t>(T) * W * sizeof(float), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
            cudaStreamSynchronize(st) != cudaSuccess) rc = -2;
      }
    }
    if (pend.y) KRN("residual_norm", sandwich_step(boundary(pend, nullptr, nullptr, dt, nullptr, T), st));
    // head: the final norm of the wanted rows, logits in fp32, greedy choice
    for (int r0 = 0; r0 < b.S && !rc; r0 += row_cap) {
      const int n = std::min(row_cap, b.S - r0);
      KRN("residual_norm", sandwich_step(boundary(Pending(), fin_w, hrow, dt, b.rows + r0, n), st));
      KRN("head", linear(linear_args(hrow, dt, head, dt, logits, DT_F32, n, V, W), st));
      KRN("argmax", argmax_f32(logits, sampled + r0, n, V, st));
      if (host_logits && cudaMemcpyAsync(host_logits + static_cast<size_t>(r0) * V, logits, static_cast<size_t>(n) * V * sizeof(float),
                                         cudaMemcpyDeviceToHost, st) != cudaSuccess) rc = -2;
    }
    if (launches) *launches += nl;
    if (rc) { set_error("Mulenex forward: %s failed with %d (%s)", failed_kernel, failed_rc, cudaGetErrorString(cudaGetLastError())); return -2; }
    return 0;
  }
};

}  // namespace

#undef KRN

std::unique_ptr<Model> make_mulenex(const JVal& config, DType dtype, std::string* err) {
  std::unique_ptr<Mulenex> m(new Mulenex(dtype));
  if (!m->parse(config, err)) return nullptr;
  return std::unique_ptr<Model>(m.release());
}

}  // namespace b200
