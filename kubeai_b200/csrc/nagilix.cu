// Nagilix: a decoder-only design on several fp32 residual streams (hyper-connections) with a gated write-back, whose
// layers mix tokens either by two mixers side by side or by a selective scan, and whose feed-forward is a mixture of
// clamped gated experts that also counts identity experts.
//
//   x_s[t]    = embed[token] + pos[p]                                  for every stream s (a learned position row)
//   sublayer  : u = sum_s in[s] x_s;  h = g * u / rms(u)  (ONE learned number g per norm);  y = f(h);
//               y <- y * sigmoid(W_rg h + b_rg);  x_j <- sum_s mix[s, j] x_s + out[j] y                       (hyper.cu)
//   parallel  = 1/2 (w_l * left(h) / rms(left(h)) + w_r * right(h) / rms(right(h)))          (branch_norm_sum)
//     left    : q = W_q h, k = W_k h pass a short causal convolution over time; the values are the convolved keys; q and k
//               are RMS-normed over the whole projection with weights and rotated (rotate-half layout, first rot.dims
//               dimensions of a head); score = q . k * scale * temp_h; a token sees the keys of its own chunk of
//               mask.size positions up to itself; the softmax denominator also holds exp(sink_h); W_o
//                                                                        (window_attention.cu: conv_qk_prep, chunk, sink)
//     right   : retention: S <- decay_h S + k v^T, o = S^T q on rotated q and k (k scaled by dim^-1/2), every head's o
//               divided by its RMS, times silu(W_g h), W_o                             (gla.cu, head_decay form with rope)
//   mamba1    : [x | z] = W_in h; x <- silu(conv(x) + b); [dt | B | C] = W_x x; d = softplus(W_dt dt + b_dt);
//               S[c, n] <- exp(d_c A[c, n]) S[c, n] + d_c x_c B_n; y_c = S[c, :] . C + D_c x_c; W_o (y * silu(z))   (ssm.cu)
//   ff        : s = softmax(W_router h) over experts + identity experts; the `top` largest s + correction are chosen,
//               weighted by s itself; expert(h) = W_down (g * sigmoid(1.702 g) * (u + 1)), g = min(W_gate h, limit),
//               u = clamp(W_up h, -limit, limit); an identity expert returns h                    (moe.cu, linear.cu)
//   logits    = head (g_f * x / rms(x)) * logit_scale,  x = sum_s x_s
//
// Per layer the kernel sequence is: the stream boundary (previous gated write-back + read + norm), ONE input projection
// for everything that reads the mixer's input (the residual gate's rows ride behind the mixer's), the mixer's own
// kernels, its output projection(s), and for the feed-forward the gate projection, the fp32 router product, routing and
// the experts.  Every size and constant comes from config.json; matrices and activations are bf16 or fp32; the streams,
// norms, softmax, router, step sizes, decays and recurrent states are fp32 either way.  A sequence's state slot holds
// the carried inputs of every convolution, the retention state of every parallel layer and the scan state of every
// mamba layer; the page pool holds keys and values of the parallel layers.
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

enum MixerKind { MIX_PARALLEL = 0, MIX_MAMBA = 1 };

struct LeftSpec {
  int heads = 0, kv_heads = 0, dim = 0, taps = 1, chunk = 0, rot_dims = 0;
  double rot_base = 10000.0;
  float scale = 1.f;
};
struct RightSpec {
  int heads = 0, dim = 0, vdim = 0, rot_dims = 0;
  double rot_base = 10000.0;
  std::vector<float> decay;
};
struct MambaSpec {
  int inner = 0, state = 0, dt_rank = 0, taps = 1;
};
struct LayerSpec {
  int kind = MIX_PARALLEL;
  LeftSpec l;
  RightSpec r;
  MambaSpec m;
  bool mlp = false;
  int experts = 0, identity = 0, top = 0, ff = 0;
  float limit = 0.f;
  // column layout of the input projection's output row
  int n_in = 0, off_qk = 0, off_rq = 0, off_rk = 0, off_rv = 0, off_rg = 0, off_x = 0, off_z = 0, off_gate = 0;
  int hv_l = 0, hv_r = 0, conv_c = 0;
  size_t conv_floats = 0, rec_floats = 0;   // the layer's part of a state slot: carried convolution inputs, recurrent state
};

struct Hyper {   // one sublayer's stream weights (device, fp32); null when the model has a single plain residual
  float *in = nullptr, *out = nullptr, *mix = nullptr;
};

struct LayerWeights {
  void* w_in = nullptr;     // [n_in, width]
  void* w_lo = nullptr;     // parallel: [width, heads * dim]   mamba: W_o [width, inner]
  void* w_ro = nullptr;     // parallel: [width, heads * vdim]
  void* w_x = nullptr;      // mamba: [dt_rank + 2 state, inner]
  void* w_dt = nullptr;     // mamba: [inner, dt_rank]
  float *norm1 = nullptr, *norm2 = nullptr;          // the norm's one number, spread over the width
  float *conv_w = nullptr, *conv_b = nullptr;        // [channels, taps], [channels]
  float *q_norm = nullptr, *k_norm = nullptr, *temp = nullptr, *sink = nullptr, *decay = nullptr, *out_l = nullptr, *out_r = nullptr;
  float *dt_b = nullptr, *A = nullptr, *Dskip = nullptr;
  float2 *rope_l = nullptr, *rope_r = nullptr;
  float *rg1_b = nullptr, *rg2_b = nullptr, *correction = nullptr;
  Hyper hc1, hc2;
  void* rg2 = nullptr;      // [width, width]
  void* router = nullptr;   // [experts + identity, width]
  void* e_gu = nullptr;     // [experts][2 ff][width]  gate rows, then up rows
  void* e_down = nullptr;   // [experts][width][ff]
  GemmPlan p_in, p_lo, p_ro, p_rg2;
  std::vector<GemmPlan> p_egu, p_edown;
  CUtensorMap xm_lo[kGemmNumBlockN], xm_ro[kGemmNumBlockN];
  bool tc_in = false, tc_lo = false, tc_ro = false, tc_rg2 = false;
};

struct LayerRun {
  void* cache = nullptr;    // parallel: [num_blocks * page][kv_heads * 2 dim]
  float* conv = nullptr;    // [slots][taps - 1][channels]: the carried inputs of the layer's convolution
  float* state = nullptr;   // [slots][...]: the retention state (heads x dim x vdim) or the scan state (inner x state)
};

bool jnum(const JVal* o, const char* k, double* out) {
  const JVal* v = o ? o->get(k) : nullptr;
  if (!v || v->type != JVal::Num) return false;
  *out = v->num;
  return true;
}

class Nagilix : public Model {
 public:
  DType dt;
  int V = 0, W = 0, ns = 1, max_pos = 0;
  bool hyper = false;     // the config names `streams`: every sublayer has stream weights
  bool gated = true;      // every sublayer's write-back passes a sigmoid gate (the checkpoint says so)
  float eps = 1e-5f, logit_scale = 1.f;
  std::vector<LayerSpec> spec;
  std::vector<LayerWeights> wts;
  std::vector<LayerRun> run;
  ModelEnv env;
  void *embed = nullptr, *pos_table = nullptr, *head = nullptr;
  float* fin_w = nullptr;
  // activations
  float* x = nullptr;            // [ns][Tcap][W]
  long long xstride = 0;
  void *h = nullptr, *inb = nullptr, *yl = nullptr, *yr = nullptr, *al = nullptr, *ar = nullptr, *xc = nullptr, *fo = nullptr, *g2 = nullptr, *hrow = nullptr;
  void *egu = nullptr, *eact = nullptr;
  float *qn = nullptr, *o32 = nullptr, *ysum = nullptr, *xdbc = nullptr, *dtp = nullptr, *scores = nullptr, *topw = nullptr, *edown = nullptr,
        *logits = nullptr, *sumbuf = nullptr;
  int *topi = nullptr, *sorted_rows = nullptr, *tile_group = nullptr, *pair_pos = nullptr, *iota = nullptr;
  int row_cap = 0, moe_cap = 0;
  void *hsorted = nullptr, *edown16 = nullptr;
  int *expert_rows = nullptr, *expert_rows_host = nullptr;
  std::vector<void*> allocs;
  float* gemm_ws = nullptr;
  int* gemm_counters = nullptr;
  CUtensorMap xm_h[kGemmNumBlockN];
  bool use_tc = false;

  explicit Nagilix(DType d) : dt(d) {}
  ~Nagilix() override {
    for (auto& w : wts) {
      if (w.tc_in) gemm_plan_destroy(&w.p_in);
      if (w.tc_lo) gemm_plan_destroy(&w.p_lo);
      if (w.tc_ro) gemm_plan_destroy(&w.p_ro);
      if (w.tc_rg2) gemm_plan_destroy(&w.p_rg2);
      for (auto& p : w.p_egu) gemm_plan_destroy(&p);
      for (auto& p : w.p_edown) gemm_plan_destroy(&p);
    }
    if (expert_rows_host) cudaFreeHost(expert_rows_host);
    for (void* p : allocs) cudaFree(p);
  }
  const char* arch() const override { return "Nagilix"; }
  int vocab() const override { return V; }
  int max_positions() const override { return max_pos; }

  size_t cache_bytes_per_block(int page) const override {
    size_t b = 0;
    for (auto& s : spec)
      if (s.kind == MIX_PARALLEL) b += static_cast<size_t>(page) * s.l.kv_heads * 2 * s.l.dim * dtype_bytes(dt);
    return b;
  }
  size_t state_bytes_per_slot() const override {
    size_t b = 0;
    for (auto& s : spec) b += (s.conv_floats + s.rec_floats) * sizeof(float);
    return b;
  }
  // a token never looks further back than the start of its chunk: pages that end before every layer's chunk can go
  int cache_window() const override {
    int w = 0;
    for (auto& s : spec) {
      if (s.kind != MIX_PARALLEL) continue;
      if (s.l.chunk <= 0) return 0;
      w = std::max(w, s.l.chunk);
    }
    return w;
  }

  // ------------------------------------------------------------ config.json
  bool parse(const JVal& c, std::string* err) {
    double d = 0;
    auto whole = [&](const JVal* o, const char* k, int lo, int* out, const std::string& where) {
      double v = 0;
      if (!jnum(o, k, &v) || v < lo || v != floor(v) || v > 2147483647.0) { *err = "config: " + where + k; return false; }
      *out = static_cast<int>(v);
      return true;
    };
    auto rotation = [&](const JVal* o, int dim, int* dims, double* base, const std::string& where) {
      const JVal* rot = o->get("rot");
      if (!rot || rot->type != JVal::Obj) return true;     // no rotation
      *dims = dim / 2 * 2;
      if (rot->get("dims") && !whole(rot, "dims", 0, dims, where + "rot.")) return false;
      double b = 0;
      if (jnum(rot, "base", &b)) *base = b;
      if (*dims > dim || *dims % 2 || !(*base > 0)) { *err = "config: " + where + "rot"; return false; }
      return true;
    };
    if (!whole(&c, "vocab", 1, &V, "") || !whole(&c, "width", 1, &W, "") || !whole(&c, "max_positions", 1, &max_pos, "")) return false;
    if (jnum(c.get("norm"), "eps", &d)) eps = static_cast<float>(d);
    if (jnum(&c, "logit_scale", &d)) logit_scale = static_cast<float>(d);
    if (const JVal* sv = c.get("streams")) {
      if (!sv->is_null()) {
        if (!whole(&c, "streams", 1, &ns, "") || ns > 8) { *err = "config: streams (1..8)"; return false; }
        hyper = true;
      }
    }
    const JVal* ls = c.get("layers");
    if (!ls || ls->type != JVal::Arr || ls->arr.empty()) { *err = "config: layers"; return false; }
    for (size_t i = 0; i < ls->arr.size(); ++i) {
      const JVal& L = ls->arr[i];
      const std::string where = "layer " + std::to_string(i) + " ";
      LayerSpec s;
      const JVal* ty = L.get("type");
      const JVal* mx = L.get("mixer");
      if (!ty || ty->type != JVal::Str) { *err = "config: " + where + "type"; return false; }
      if (!mx || mx->type != JVal::Obj) { *err = "config: " + where + "mixer"; return false; }
      if (ty->str == "parallel") {
        s.kind = MIX_PARALLEL;
        const JVal* lf = mx->get("left");
        const JVal* rt = mx->get("right");
        if (!lf || lf->type != JVal::Obj || !rt || rt->type != JVal::Obj) { *err = "config: " + where + "mixer.left / mixer.right"; return false; }
        LeftSpec& l = s.l;
        int vdim = 0;
        if (!whole(lf, "heads", 1, &l.heads, where + "left.") || !whole(lf, "dim", 1, &l.dim, where + "left.")) return false;
        l.kv_heads = l.heads;
        if (lf->get("kv_heads") && !whole(lf, "kv_heads", 1, &l.kv_heads, where + "left.")) return false;
        if (l.heads % l.kv_heads) { *err = "config: " + where + "left.heads is no multiple of kv_heads"; return false; }
        vdim = l.dim;
        if (lf->get("vdim") && !whole(lf, "vdim", 1, &vdim, where + "left.")) return false;
        if (vdim != l.dim) { *err = "config: " + where + "left.vdim differs from dim: this attention takes its values from the keys"; return false; }
        if (l.dim > 256) { *err = "config: " + where + "left.dim above 256"; return false; }
        if (lf->get("conv") && !lf->get("conv")->is_null() && !whole(lf, "conv", 1, &l.taps, where + "left.")) return false;
        l.scale = 1.0f / sqrtf(static_cast<float>(l.dim));
        if (jnum(lf, "scale", &d)) l.scale = static_cast<float>(d);
        if (const JVal* mk = lf->get("mask"))
          if (mk->type == JVal::Obj && !whole(mk, "size", 1, &l.chunk, where + "left.mask.")) return false;
        if (!rotation(lf, l.dim, &l.rot_dims, &l.rot_base, where + "left.")) return false;
        RightSpec& r = s.r;
        if (!whole(rt, "heads", 1, &r.heads, where + "right.") || !whole(rt, "dim", 1, &r.dim, where + "right.") || !whole(rt, "vdim", 1, &r.vdim, where + "right.")) return false;
        if (r.dim > 1024) { *err = "config: " + where + "right.dim above 1024"; return false; }
        if (!rotation(rt, r.dim, &r.rot_dims, &r.rot_base, where + "right.")) return false;
        const JVal* dc = rt->get("decay");
        if (dc && dc->type == JVal::Num) r.decay.assign(r.heads, static_cast<float>(dc->num));
        else if (dc && dc->type == JVal::Arr && static_cast<int>(dc->arr.size()) == r.heads) {
          for (auto& v : dc->arr) {
            if (v.type != JVal::Num) { *err = "config: " + where + "right.decay"; return false; }
            r.decay.push_back(static_cast<float>(v.num));
          }
        } else { *err = "config: " + where + "right.decay (one number per head)"; return false; }
      } else if (ty->str == "mamba1") {
        s.kind = MIX_MAMBA;
        MambaSpec& m = s.m;
        if (!whole(mx, "inner", 1, &m.inner, where + "mixer.") || !whole(mx, "state", 1, &m.state, where + "mixer.") ||
            !whole(mx, "dt_rank", 1, &m.dt_rank, where + "mixer.")) return false;
        if (mx->get("conv") && !mx->get("conv")->is_null() && !whole(mx, "conv", 1, &m.taps, where + "mixer.")) return false;
        if (m.state > 256) { *err = "config: " + where + "mixer.state above 256"; return false; }
      } else { *err = "config: unknown mixer \"" + ty->str + "\""; return false; }
      const JVal* mlp = L.get("mlp");
      if (mlp && mlp->type == JVal::Obj) {
        const JVal* kind = mlp->get("kind");
        if (!kind || kind->type != JVal::Str || kind->str != "moe") { *err = "config: " + where + "mlp.kind (moe)"; return false; }
        s.mlp = true;
        const JVal* ex = mlp->get("expert");
        const JVal* ro = mlp->get("router");
        if (!whole(ex, "ff", 1, &s.ff, where + "mlp.expert.") || !whole(ro, "experts", 0, &s.experts, where + "mlp.router.") ||
            !whole(ro, "top", 1, &s.top, where + "mlp.router.")) return false;
        if (ro->get("identity") && !whole(ro, "identity", 0, &s.identity, where + "mlp.router.")) return false;
        if (s.top > s.experts + s.identity) { *err = "config: " + where + "mlp.router.top above the number of experts"; return false; }
        s.limit = INFINITY;
        if (jnum(ex, "limit", &d)) s.limit = static_cast<float>(d);
      }
      layout(s);
      spec.push_back(s);
    }
    run.resize(spec.size());
    return true;
  }

  static int up8(int v) { return (v + 7) / 8 * 8; }
  void layout(LayerSpec& s) {
    int at = 0;
    auto block = [&](int* off, int n) { *off = at; at = up8(at + n); };   // every block starts 16-byte aligned
    if (s.kind == MIX_PARALLEL) {
      s.conv_c = (s.l.heads + s.l.kv_heads) * s.l.dim;
      block(&s.off_qk, s.conv_c);       // queries, then keys: one run of convolved channels
      block(&s.off_rq, s.r.heads * s.r.dim);
      block(&s.off_rk, s.r.heads * s.r.dim);
      block(&s.off_rv, s.r.heads * s.r.vdim);
      block(&s.off_rg, s.r.heads * s.r.vdim);
      s.hv_l = s.l.heads * s.l.dim;
      s.hv_r = s.r.heads * s.r.vdim;
      s.conv_floats = static_cast<size_t>(s.l.taps - 1) * s.conv_c;
      s.rec_floats = static_cast<size_t>(s.r.heads) * s.r.dim * s.r.vdim;
    } else {
      s.conv_c = s.m.inner;
      block(&s.off_x, s.m.inner);
      block(&s.off_z, s.m.inner);
      s.conv_floats = static_cast<size_t>(s.m.taps - 1) * s.conv_c;
      s.rec_floats = static_cast<size_t>(s.m.inner) * s.m.state;
    }
    block(&s.off_gate, gated ? W : 0);   // the residual gate reads the same input: its rows ride in the same product
    s.n_in = at;
  }

  // what only the checkpoint says: whether the sublayers' write-backs are gated
  int inspect(const CheckpointReader& ck, std::string* err) override {
    gated = ck.has("l0.rg1");
    for (auto& s : spec) layout(s);
    return 0;
  }

  template <typename P>
  int dalloc(P** p, size_t bytes) {
    void* q = nullptr;
    if (cudaMalloc(&q, std::max<size_t>(bytes, 16)) != cudaSuccess) { set_error("Nagilix: device allocation of %zu bytes failed", bytes); return -3; }
    cudaMemsetAsync(q, 0, std::max<size_t>(bytes, 16), env.stream);
    allocs.push_back(q);
    *p = static_cast<P*>(q);
    return 0;
  }

  int init(const ModelEnv& e) override {
    env = e;
    const size_t es = dtype_bytes(dt);
    wts.resize(spec.size());
    int max_in = 8, max_hvl = 8, max_hvr = 8, max_qn = 1, max_e = 1, max_top = 1, max_ff = 1, max_inner = 8, max_xdbc = 1;
    bool any_moe = false, any_par = false, any_mamba = false;
    for (auto& s : spec) {
      max_in = std::max(max_in, s.n_in);
      if (s.kind == MIX_PARALLEL) {
        any_par = true;
        max_hvl = std::max(max_hvl, s.hv_l); max_hvr = std::max(max_hvr, s.hv_r); max_qn = std::max(max_qn, s.hv_l);
      } else {
        any_mamba = true;
        max_inner = std::max(max_inner, s.m.inner); max_xdbc = std::max(max_xdbc, s.m.dt_rank + 2 * s.m.state);
      }
      if (s.mlp) {
        any_moe = true;
        max_e = std::max(max_e, s.experts + s.identity); max_top = std::max(max_top, s.top); max_ff = std::max(max_ff, s.ff);
      }
    }
    int rc = 0;
    auto mat = [&](void** p, size_t rows, size_t cols) { return dalloc(p, rows * cols * es); };
    auto vec = [&](float** p, size_t n) { return dalloc(p, n * sizeof(float)); };
    rc |= mat(&embed, V, W) | mat(&pos_table, max_pos, W) | mat(&head, V, W) | vec(&fin_w, W);
    for (size_t i = 0; i < spec.size() && !rc; ++i) {
      const LayerSpec& s = spec[i];
      if (s.kind == MIX_PARALLEL) rc |= dalloc(&run[i].cache, static_cast<size_t>(e.num_blocks) * e.page * s.l.kv_heads * 2 * s.l.dim * es);
      rc |= dalloc(&run[i].conv, static_cast<size_t>(e.num_slots) * s.conv_floats * sizeof(float)) |
            dalloc(&run[i].state, static_cast<size_t>(e.num_slots) * s.rec_floats * sizeof(float));
    }
    if (rc) return rc;
    for (size_t i = 0; i < spec.size() && !rc; ++i) {
      const LayerSpec& s = spec[i];
      LayerWeights& w = wts[i];
      rc |= mat(&w.w_in, s.n_in, W) | vec(&w.norm1, W);
      if (gated) rc |= vec(&w.rg1_b, W);
      if (hyper) rc |= vec(&w.hc1.in, ns) | vec(&w.hc1.out, ns) | vec(&w.hc1.mix, static_cast<size_t>(ns) * ns);
      if (s.kind == MIX_PARALLEL) {
        rc |= mat(&w.w_lo, W, s.hv_l) | mat(&w.w_ro, W, s.hv_r) | vec(&w.q_norm, s.hv_l) | vec(&w.k_norm, s.l.kv_heads * s.l.dim) | vec(&w.temp, s.l.heads) |
              vec(&w.sink, s.l.heads) | vec(&w.decay, s.r.heads) | vec(&w.out_l, W) | vec(&w.out_r, W);
        if (s.l.taps > 1) rc |= vec(&w.conv_w, static_cast<size_t>(s.conv_c) * s.l.taps);
        if (!rc && cudaMemcpyAsync(w.decay, s.r.decay.data(), s.r.heads * sizeof(float), cudaMemcpyHostToDevice, e.stream) != cudaSuccess) rc = -2;
        if (s.l.rot_dims > 0) {
          rc |= dalloc(&w.rope_l, static_cast<size_t>(e.max_model_len) * (s.l.rot_dims / 2) * sizeof(float2));
          if (!rc && rope_table_yarn(w.rope_l, e.max_model_len, s.l.rot_dims, s.l.rot_base, nullptr, e.stream)) rc = -2;
        }
        if (s.r.rot_dims > 0) {
          rc |= dalloc(&w.rope_r, static_cast<size_t>(e.max_model_len) * (s.r.rot_dims / 2) * sizeof(float2));
          if (!rc && rope_table_yarn(w.rope_r, e.max_model_len, s.r.rot_dims, s.r.rot_base, nullptr, e.stream)) rc = -2;
        }
      } else {
        const MambaSpec& m = s.m;
        rc |= mat(&w.w_lo, W, m.inner) | mat(&w.w_x, m.dt_rank + 2 * m.state, m.inner) | mat(&w.w_dt, m.inner, m.dt_rank) | vec(&w.dt_b, m.inner) |
              vec(&w.A, static_cast<size_t>(m.inner) * m.state) | vec(&w.Dskip, m.inner) | vec(&w.conv_w, static_cast<size_t>(m.inner) * m.taps) |
              vec(&w.conv_b, m.inner);
      }
      if (s.mlp) {
        rc |= vec(&w.norm2, W) | mat(&w.router, s.experts + s.identity, W) | vec(&w.correction, s.experts + s.identity) |
              mat(&w.e_gu, static_cast<size_t>(std::max(s.experts, 1)) * 2 * s.ff, W) | mat(&w.e_down, static_cast<size_t>(std::max(s.experts, 1)) * W, s.ff);
        if (gated) rc |= mat(&w.rg2, W, W) | vec(&w.rg2_b, W);
        if (hyper) rc |= vec(&w.hc2.in, ns) | vec(&w.hc2.out, ns) | vec(&w.hc2.mix, static_cast<size_t>(ns) * ns);
      }
    }
    if (rc) return rc;
    const size_t T = e.Tcap;
    row_cap = static_cast<int>(std::min<size_t>(T, 256));
    xstride = static_cast<long long>(T) * W;
    rc |= dalloc(&x, static_cast<size_t>(ns) * T * W * sizeof(float)) | mat(&h, T, W) | mat(&inb, T, max_in) | mat(&al, T, W) | mat(&hrow, row_cap, W) |
          dalloc(&logits, static_cast<size_t>(row_cap) * V * sizeof(float));
    rc |= mat(&yl, T, std::max(max_hvl, max_inner));
    if (any_par) rc |= mat(&yr, T, max_hvr) | mat(&ar, T, W) | dalloc(&qn, T * max_qn * sizeof(float)) | dalloc(&o32, T * max_hvr * sizeof(float)) |
                       dalloc(&ysum, T * W * sizeof(float));
    if (any_mamba) rc |= mat(&xc, T, max_inner) | dalloc(&xdbc, T * max_xdbc * sizeof(float)) | dalloc(&dtp, T * max_inner * sizeof(float));
    if (any_moe) {
      moe_cap = static_cast<int>((T * max_top + 63) / 64 * 64) + max_e * 64;
      rc |= mat(&fo, T, W) | dalloc(&scores, T * max_e * sizeof(float)) | dalloc(&topw, T * max_top * sizeof(float)) | dalloc(&topi, T * max_top * sizeof(int)) |
            dalloc(&sorted_rows, static_cast<size_t>(moe_cap) * sizeof(int)) | dalloc(&tile_group, static_cast<size_t>(moe_cap / 64) * sizeof(int)) |
            dalloc(&pair_pos, T * max_top * sizeof(int)) | mat(&egu, moe_cap, 2 * static_cast<size_t>(max_ff)) | mat(&eact, moe_cap, max_ff) |
            dalloc(&edown, static_cast<size_t>(moe_cap) * W * sizeof(float)) | dalloc(&iota, static_cast<size_t>(64) * sizeof(int));
      if (gated) rc |= mat(&g2, T, W);
      if (!rc) {
        int hi[64];
        for (int i = 0; i < 64; ++i) hi[i] = i;
        if (cudaMemcpyAsync(iota, hi, sizeof(hi), cudaMemcpyHostToDevice, e.stream) != cudaSuccess || cudaStreamSynchronize(e.stream) != cudaSuccess) rc = -2;
      }
    }
    if (rc) return rc;
    register_tensors();
    rc = setup_tc();
    if (rc) return rc;
    return cudaStreamSynchronize(e.stream) == cudaSuccess ? 0 : -2;
  }

  // The projections of a bf16 model run on the tcgen05 pair GEMM (gemm2_tcgen05.cu) where their shapes allow it (K % 8 == 0):
  // the input projection, the output projections, the feed-forward's gate projection and every expert for steps large
  // enough to sort rows per expert.  The thin products with fp32 results (router, [dt | B | C], the step sizes) and every
  // projection of an fp32 model stay on linear.cu.  B200_NG_TC=0 keeps everything there (A/B knob).
  int setup_tc() {
    const char* ev = getenv("B200_NG_TC");
    use_tc = dt == DT_BF16 && !(ev && atoi(ev) == 0) && W % 8 == 0 && gemm_variant() == 2;
    if (!use_tc) return 0;
    int maxN = W;
    for (auto& s : spec) maxN = std::max(std::max(maxN, s.n_in), 2 * s.ff);
    const size_t ws_bytes = std::max(gemm_workspace_bytes(env.sms), gemm_deferred_ws_bytes(env.sms));
    if (dalloc(&gemm_ws, ws_bytes)) return -3;
    const size_t n_counters = 2ull * (maxN / 128 + 2) * (env.Tcap / 32 + 2);
    if (dalloc(&gemm_counters, n_counters * sizeof(int))) return -3;
    const int bns[kGemmNumBlockN] = {32, 64, 128, 256, 512};
    for (int i = 0; i < kGemmNumBlockN; ++i)
      if (gemm_make_x_map(&xm_h[i], h, env.Tcap, W, W, bns[i])) { use_tc = false; return 0; }
    bool any_expert_tc = false;
    for (size_t i = 0; i < spec.size(); ++i) {
      const LayerSpec& s = spec[i];
      LayerWeights& w = wts[i];
      w.tc_in = gemm_plan_init(&w.p_in, w.w_in, s.n_in, W, W, gemm_ws, gemm_counters, env.sms) == 0;
      if (w.tc_in) w.p_in.ws_bytes = ws_bytes;
      const int k_lo = s.kind == MIX_PARALLEL ? s.hv_l : s.m.inner;
      w.tc_lo = k_lo % 8 == 0 && gemm_plan_init(&w.p_lo, w.w_lo, W, k_lo, k_lo, gemm_ws, gemm_counters, env.sms) == 0;
      for (int j = 0; j < kGemmNumBlockN && w.tc_lo; ++j)
        if (gemm_make_x_map(&w.xm_lo[j], yl, env.Tcap, k_lo, k_lo, bns[j])) w.tc_lo = false;
      if (w.tc_lo) w.p_lo.ws_bytes = ws_bytes;
      if (s.kind == MIX_PARALLEL) {
        w.tc_ro = s.hv_r % 8 == 0 && gemm_plan_init(&w.p_ro, w.w_ro, W, s.hv_r, s.hv_r, gemm_ws, gemm_counters, env.sms) == 0;
        for (int j = 0; j < kGemmNumBlockN && w.tc_ro; ++j)
          if (gemm_make_x_map(&w.xm_ro[j], yr, env.Tcap, s.hv_r, s.hv_r, bns[j])) w.tc_ro = false;
        if (w.tc_ro) w.p_ro.ws_bytes = ws_bytes;
      }
      if (s.mlp && gated) {
        w.tc_rg2 = gemm_plan_init(&w.p_rg2, w.rg2, W, W, W, gemm_ws, gemm_counters, env.sms) == 0;
        if (w.tc_rg2) w.p_rg2.ws_bytes = ws_bytes;
      }
      if (s.mlp && s.experts > 0 && s.ff % 8 == 0) {
        w.p_egu.resize(s.experts);
        w.p_edown.resize(s.experts);
        bool ok = true;
        for (int e = 0; e < s.experts && ok; ++e) {
          ok = gemm_plan_init(&w.p_egu[e], static_cast<bf16*>(w.e_gu) + static_cast<size_t>(e) * 2 * s.ff * W, 2 * s.ff, W, W, gemm_ws, gemm_counters, env.sms) == 0 &&
               gemm_plan_init(&w.p_edown[e], static_cast<bf16*>(w.e_down) + static_cast<size_t>(e) * W * s.ff, W, s.ff, s.ff, gemm_ws, gemm_counters, env.sms) == 0;
          w.p_egu[e].ws_bytes = w.p_edown[e].ws_bytes = ws_bytes;
        }
        if (!ok) { w.p_egu.clear(); w.p_edown.clear(); }
        else any_expert_tc = true;
      }
    }
    if (any_expert_tc) {
      int max_e = 1;
      for (auto& s : spec) max_e = std::max(max_e, s.experts + s.identity);
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
    for (size_t i = 0; i < spec.size(); ++i) reg("l" + std::to_string(i) + ".w_in", wts[i].w_in, static_cast<size_t>(spec[i].n_in) * W * es);
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
  int putf(float* dst, const std::vector<float>& src) {
    return cudaMemcpy(dst, src.data(), src.size() * sizeof(float), cudaMemcpyHostToDevice) == cudaSuccess ? 0 : -2;
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
    // a norm's one number, spread over the width (times `mult`)
#define NORM1(name, dst, mult) do { if (!get(name, 1, 1)) return -4; const float g_ = v[0] * (mult); v.assign(W, g_); rc |= putf(dst, v); } while (0)
#define HC(prefix, hc) do { if (hyper) { VEC(prefix + "in", hc.in, ns); VEC(prefix + "out", hc.out, ns); if (!get(prefix + "mix", ns, ns)) return -4; rc |= putf(hc.mix, v); } } while (0)
    MAT("embed", embed, W, 0, 0, V, W);
    MAT("pos", pos_table, W, 0, 0, max_pos, W);
    MAT("head", head, W, 0, 0, V, W);
    NORM1("final.norm", fin_w, logit_scale);   // the scale of the logits rides in the last norm's number
    for (size_t i = 0; i < spec.size(); ++i) {
      const LayerSpec& s = spec[i];
      LayerWeights& w = wts[i];
      const std::string p = "l" + std::to_string(i) + ".", mx = p + "mix.", lf = mx + "left.", rt = mx + "right.", f = p + "mlp.";
      NORM1(p + "norm1", w.norm1, 1.0f);
      HC(p + "hc1.", w.hc1);
      if (gated) { MAT(p + "rg1", w.w_in, W, s.off_gate, 0, W, W); VEC(p + "rg1.b", w.rg1_b, W); }
      if (s.kind == MIX_PARALLEL) {
        const int HD = s.hv_l, GD = s.l.kv_heads * s.l.dim;
        MAT(lf + "q", w.w_in, W, s.off_qk, 0, HD, W);
        MAT(lf + "k", w.w_in, W, s.off_qk + HD, 0, GD, W);
        if (s.l.taps > 1) {
          std::vector<float> cw(static_cast<size_t>(s.conv_c) * s.l.taps);
          if (!get(lf + "q.conv", HD, s.l.taps)) return -4;
          std::copy(v.begin(), v.end(), cw.begin());
          if (!get(lf + "k.conv", GD, s.l.taps)) return -4;
          std::copy(v.begin(), v.end(), cw.begin() + static_cast<size_t>(HD) * s.l.taps);
          rc |= putf(w.conv_w, cw);
        }
        VEC(lf + "q.norm", w.q_norm, HD);
        VEC(lf + "k.norm", w.k_norm, GD);
        VEC(lf + "temp", w.temp, s.l.heads);
        VEC(lf + "sink", w.sink, s.l.heads);
        MAT(lf + "o", w.w_lo, HD, 0, 0, W, HD);
        MAT(rt + "q", w.w_in, W, s.off_rq, 0, s.r.heads * s.r.dim, W);
        MAT(rt + "k", w.w_in, W, s.off_rk, 0, s.r.heads * s.r.dim, W);
        MAT(rt + "v", w.w_in, W, s.off_rv, 0, s.hv_r, W);
        MAT(rt + "g", w.w_in, W, s.off_rg, 0, s.hv_r, W);
        MAT(rt + "o", w.w_ro, s.hv_r, 0, 0, W, s.hv_r);
        VEC(lf + "out", w.out_l, W);
        VEC(rt + "out", w.out_r, W);
      } else {
        const MambaSpec& m = s.m;
        if (!get(mx + "in", 2 * m.inner, W)) return -4;
        {
          std::vector<float> top(v.begin(), v.begin() + static_cast<size_t>(m.inner) * W), bot(v.begin() + static_cast<size_t>(m.inner) * W, v.end());
          rc |= put(w.w_in, W, s.off_x, 0, top, m.inner, W) | put(w.w_in, W, s.off_z, 0, bot, m.inner, W);
        }
        if (!get(mx + "conv", m.inner, m.taps)) return -4;
        rc |= putf(w.conv_w, v);
        VEC(mx + "conv.b", w.conv_b, m.inner);
        MAT(mx + "x", w.w_x, m.inner, 0, 0, m.dt_rank + 2 * m.state, m.inner);
        MAT(mx + "dt", w.w_dt, m.dt_rank, 0, 0, m.inner, m.dt_rank);
        VEC(mx + "dt.b", w.dt_b, m.inner);
        if (!get(mx + "A_log", m.inner, m.state)) return -4;
        for (auto& a : v) a = -expf(a);           // A = -exp(A_log), once
        rc |= putf(w.A, v);
        VEC(mx + "D", w.Dskip, m.inner);
        MAT(mx + "o", w.w_lo, m.inner, 0, 0, W, m.inner);
      }
      if (!s.mlp) continue;
      NORM1(p + "norm2", w.norm2, 1.0f);
      HC(p + "hc2.", w.hc2);
      if (gated) { MAT(p + "rg2", w.rg2, W, 0, 0, W, W); VEC(p + "rg2.b", w.rg2_b, W); }
      MAT(f + "router", w.router, W, 0, 0, s.experts + s.identity, W);
      VEC(f + "correction", w.correction, s.experts + s.identity);
      for (int e = 0; e < s.experts; ++e) {
        const std::string ep = f + "e" + std::to_string(e) + ".";
        MAT(ep + "gate", w.e_gu, W, static_cast<size_t>(e) * 2 * s.ff, 0, s.ff, W);
        MAT(ep + "up", w.e_gu, W, static_cast<size_t>(e) * 2 * s.ff + s.ff, 0, s.ff, W);
        MAT(ep + "down", w.e_down, s.ff, static_cast<size_t>(e) * W, 0, W, s.ff);
      }
    }
#undef MAT
#undef VEC
#undef NORM1
#undef HC
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
    M(embed, static_cast<size_t>(V) * W, 1.f);
    M(pos_table, static_cast<size_t>(max_pos) * W, 0.3f);
    M(head, static_cast<size_t>(V) * W, sw);
    F(fin_w, W, 0.f, logit_scale);
    for (size_t i = 0; i < spec.size(); ++i) {
      const LayerSpec& s = spec[i];
      LayerWeights& w = wts[i];
      M(w.w_in, static_cast<size_t>(s.n_in) * W, sw);
      F(w.norm1, W, 0.f, 1.f); F(w.rg1_b, W, 0.5f, 0.5f);
      F(w.hc1.in, ns, 0.1f, 1.0f / ns); F(w.hc1.out, ns, 0.1f, 0.5f); F(w.hc1.mix, static_cast<size_t>(ns) * ns, 0.1f, 1.0f / ns);
      if (s.kind == MIX_PARALLEL) {
        M(w.w_lo, static_cast<size_t>(W) * s.hv_l, 1.7f / sqrtf(static_cast<float>(s.hv_l)));
        M(w.w_ro, static_cast<size_t>(W) * s.hv_r, 1.7f / sqrtf(static_cast<float>(s.hv_r)));
        F(w.conv_w, static_cast<size_t>(s.conv_c) * s.l.taps, 0.5f, 0.3f);
        F(w.q_norm, s.hv_l, 0.1f, 1.f); F(w.k_norm, s.l.kv_heads * s.l.dim, 0.1f, 1.f);
        F(w.temp, s.l.heads, 0.2f, 1.f); F(w.sink, s.l.heads, 1.f, 0.f);
        F(w.out_l, W, 0.1f, 1.f); F(w.out_r, W, 0.1f, 1.f);
      } else {
        const MambaSpec& m = s.m;
        M(w.w_lo, static_cast<size_t>(W) * m.inner, 1.7f / sqrtf(static_cast<float>(m.inner)));
        M(w.w_x, static_cast<size_t>(m.dt_rank + 2 * m.state) * m.inner, 1.7f / sqrtf(static_cast<float>(m.inner)));
        M(w.w_dt, static_cast<size_t>(m.inner) * m.dt_rank, 1.7f / sqrtf(static_cast<float>(m.dt_rank)));
        F(w.dt_b, m.inner, 1.f, -3.f);
        F(w.A, static_cast<size_t>(m.inner) * m.state, 2.f, -2.5f);    // negative
        F(w.Dskip, m.inner, 0.2f, 1.f);
        F(w.conv_w, static_cast<size_t>(m.inner) * m.taps, 0.5f, 0.3f); F(w.conv_b, m.inner, 0.1f, 0.f);
      }
      if (!s.mlp) continue;
      F(w.norm2, W, 0.f, 1.f); F(w.rg2_b, W, 0.5f, 0.5f);
      F(w.hc2.in, ns, 0.1f, 1.0f / ns); F(w.hc2.out, ns, 0.1f, 0.5f); F(w.hc2.mix, static_cast<size_t>(ns) * ns, 0.1f, 1.0f / ns);
      M(w.rg2, static_cast<size_t>(W) * W, sw);
      M(w.router, static_cast<size_t>(s.experts + s.identity) * W, sw);
      F(w.correction, s.experts + s.identity, 0.01f, 0.f);
      M(w.e_gu, static_cast<size_t>(s.experts) * 2 * s.ff * W, sw);
      M(w.e_down, static_cast<size_t>(s.experts) * W * s.ff, 1.7f / sqrtf(static_cast<float>(s.ff)));
    }
    if (rc) return -2;
    return cudaStreamSynchronize(st) == cudaSuccess ? 0 : -2;
  }

  // ------------------------------------------------------------ forward
  int project(const GemmPlan& plan, bool tc, const CUtensorMap* xm, const void* X, const void* Wm, void* Y, int T, int N, int K) {
    if (tc) {
      const int bn = gemm_block_n_for(T);
      return gemm_run(plan, xm[gemm_block_n_index(bn)], bn, Y, N, T, env.stream);
    }
    return linear(linear_args(X, dt, Wm, dt, Y, dt, T, N, K), env.stream);
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

  // the write-back of the last sublayer, still to be applied by the next stream kernel: its result, its stream weights and its gate
  struct Pending {
    const void* y = nullptr; DType ty = DT_F32;
    const Hyper* hc = nullptr;
    const void* gate = nullptr; int ldg = 0; const float* gate_bias = nullptr;
  };
  HyperArgs boundary(const Pending& p, const float* in, const float* norm_w, void* out, DType to, const int* row_index, int rows) {
    HyperArgs a;
    a.x = x; a.streams = ns; a.stream_stride = xstride;
    a.y = p.y; a.ty = p.ty;
    a.mix = p.hc ? p.hc->mix : nullptr; a.out = p.hc ? p.hc->out : nullptr;
    a.in = in; a.norm_w = norm_w; a.eps = eps;
    a.h = out; a.th = to; a.row_index = row_index; a.rows = rows; a.W = W;
    a.gate = p.gate; a.tg = dt; a.ldg = p.ldg; a.gate_bias = p.gate_bias;
    return a;
  }

  int mix_parallel(const LayerSpec& s, const LayerWeights& w, const LayerRun& r, const StepBatch& b, int64_t& nl) {
    cudaStream_t st = env.stream;
    const int T = b.T;
    int rc = 0;
    const size_t es = dtype_bytes(dt);
    auto col = [&](void* base, size_t off) { return static_cast<void*>(static_cast<uint8_t*>(base) + off * es); };
    // left: convolution, norm over the whole projection, rotation, temperature, cache row (values = convolved keys)
    ConvQkPrepArgs qp;
    qp.qk = col(inb, s.off_qk); qp.ld = s.n_in; qp.t = dt;
    qp.conv_w = s.l.taps > 1 ? w.conv_w : nullptr; qp.taps = s.l.taps; qp.conv_state = r.conv;
    qp.q_norm_w = w.q_norm; qp.k_norm_w = w.k_norm; qp.eps = eps;
    qp.rope = w.rope_l; qp.rot_dims = s.l.rot_dims; qp.q_head_scale = w.temp;
    qp.positions = b.pos; qp.slots = b.slots; qp.seq_of_tok = b.seq_of_tok; qp.seqs = b.seqs;
    qp.qn = qn; qp.cache = r.cache;
    qp.T = T; qp.heads = s.l.heads; qp.kv_heads = s.l.kv_heads; qp.dim = s.l.dim;
    KRN("conv_qk_prep", conv_qk_prep(qp, st));
    if (s.l.taps > 1) {
      ShortConvArgs cc = {};
      cc.u = qp.qk; cc.ldu = s.n_in; cc.t = dt; cc.state = r.conv;
      cc.seq_of_tok = b.seq_of_tok; cc.seqs = b.seqs; cc.nseq = b.nseq; cc.T = T; cc.C = s.conv_c; cc.taps = s.l.taps;
      KRN("conv_carry", short_conv_carry(cc, st));
    }
    WindowAttnArgs wa;
    wa.qn = qn; wa.cache = r.cache; wa.t = dt; wa.positions = b.pos; wa.seq_of_tok = b.seq_of_tok; wa.block_tables = b.btab;
    wa.max_blocks = b.max_blocks; wa.page = env.page;
    wa.gate = nullptr; wa.ldg = 0; wa.out_scale = 1.f; wa.y = yl; wa.ldy = s.hv_l;
    wa.T = T; wa.heads = s.l.heads; wa.kv_heads = s.l.kv_heads; wa.dim = s.l.dim; wa.vdim = s.l.dim;
    wa.window = env.max_model_len; wa.keep_first = 0; wa.scale = s.l.scale;
    wa.seqs = b.seqs; wa.nseq = b.nseq; wa.max_ctx = b.max_ctx;
    wa.chunk = s.l.chunk; wa.sink = w.sink;
    KRN("chunk_attention", window_attention(wa, st));
    // right: retention on rotated queries and keys, per-head norm, SiLU gate
    GlaArgs g;
    g.qkv = inb; g.t = dt; g.ld = s.n_in; g.q_off = s.off_rq; g.k_off = s.off_rk; g.v_off = s.off_rv;
    g.z = nullptr; g.z_bias = nullptr; g.inv_tau = 1.f; g.q_scale = 1.f; g.T = T;
    g.states = r.state; g.seqs = b.seqs; g.nseq = b.nseq;
    g.heads = s.r.heads; g.dim = s.r.dim; g.vdim = s.r.vdim; g.o = o32;
    g.head_decay = w.decay;
    g.rope = w.rope_r; g.rot_dims = s.r.rot_dims; g.k_scale = 1.0f / sqrtf(static_cast<float>(s.r.dim));
    KRN("retention_scan", gla_scan(g, st));
    OutGateArgs og;
    og.o = o32; og.g = col(inb, s.off_rg); og.ldg = s.n_in; og.w = nullptr; og.eps = eps;
    og.y = yr; og.ldy = s.hv_r; og.t = dt; og.T = T; og.heads = s.r.heads; og.vdim = s.r.vdim;
    og.joint = false; og.gate_act = GATE_SILU; og.out_scale = 1.f;
    KRN("retention_out_gate", recurrent_out_gate(og, st));
    KRN("proj_out", project(w.p_lo, w.tc_lo, w.xm_lo, yl, w.w_lo, al, T, W, s.hv_l));
    KRN("proj_out", project(w.p_ro, w.tc_ro, w.xm_ro, yr, w.w_ro, ar, T, W, s.hv_r));
    BranchNormArgs bn = {al, ar, dt, w.out_l, w.out_r, eps, 0.5f, ysum, DT_F32, T, W};
    KRN("branch_norm_sum", branch_norm_sum(bn, st));
    return rc;
  }

  int mix_mamba(const LayerSpec& s, const LayerWeights& w, const LayerRun& r, const StepBatch& b, int64_t& nl) {
    cudaStream_t st = env.stream;
    const int T = b.T;
    const MambaSpec& m = s.m;
    int rc = 0;
    const size_t es = dtype_bytes(dt);
    auto col = [&](void* base, size_t off) { return static_cast<void*>(static_cast<uint8_t*>(base) + off * es); };
    ShortConvArgs cc = {};
    cc.u = col(inb, s.off_x); cc.ldu = s.n_in; cc.t = dt; cc.w = w.conv_w; cc.bias = w.conv_b; cc.act = CONV_SILU;
    cc.y = xc; cc.ldy = m.inner; cc.ty = dt; cc.state = r.conv;
    cc.seq_of_tok = b.seq_of_tok; cc.seqs = b.seqs; cc.nseq = b.nseq; cc.T = T; cc.C = m.inner; cc.taps = m.taps;
    KRN("short_conv", short_conv(cc, st));
    KRN("conv_carry", short_conv_carry(cc, st));
    // [dt | B | C] and the step sizes' pre-activations leave their products in fp32
    const int nx = m.dt_rank + 2 * m.state;
    KRN("ssm_x_proj", linear(linear_args(xc, dt, w.w_x, dt, xdbc, DT_F32, T, nx, m.inner), st));
    LinearArgs dl = linear_args(xdbc, DT_F32, w.w_dt, dt, dtp, DT_F32, T, m.inner, m.dt_rank);
    dl.ldx = nx; dl.bias = w.dt_b;
    KRN("ssm_dt_proj", linear(dl, st));
    SelectiveScanArgs sa;
    sa.x = xc; sa.ldx = m.inner; sa.z = col(inb, s.off_z); sa.ldz = s.n_in; sa.t = dt;
    sa.dt = dtp; sa.lddt = m.inner; sa.bc = xdbc; sa.ldbc = nx; sa.b_off = m.dt_rank; sa.c_off = m.dt_rank + m.state;
    sa.A = w.A; sa.D = w.Dskip; sa.states = r.state;
    sa.seqs = b.seqs; sa.nseq = b.nseq; sa.y = yl; sa.ldy = m.inner; sa.inner = m.inner; sa.state = m.state;
    KRN("selective_scan", selective_scan(sa, st));
    KRN("proj_out", project(w.p_lo, w.tc_lo, w.xm_lo, yl, w.w_lo, al, T, W, m.inner));
    return rc;
  }

  int moe(const LayerSpec& s, const LayerWeights& w, int T, int64_t& nl) {
    cudaStream_t st = env.stream;
    int rc = 0;
    const int ne = s.experts + s.identity;    // router outputs: the experts, then the identity experts
    KRN("moe_router", linear(linear_args(h, dt, w.router, dt, scores, DT_F32, T, ne, W), st));
    KRN("moe_route", moe_route(scores, topi, topw, T, ne, 1, 1, s.top, st, MOE_SOFTMAX, ne, w.correction));
    const long long gu_stride = 2ll * s.ff * W, down_stride = static_cast<long long>(W) * s.ff;
    static const int moe_tc_min = [] { const char* e = getenv("B200_NG_MOE_TC_MIN_T"); return e ? atoi(e) : 256; }();   // A/B knob
    const bool per_expert = !w.p_egu.empty() && T >= moe_tc_min;
    if (s.experts == 0) {
      // nothing but identity experts: the output is the input times the sum of the chosen weights
      KRN("moe_combine", moe_combine_identity(h, dt, iota, topw, topi, 0, h, fo, dt, T, s.top, W, st));
      return rc;
    }
    if (T * s.top <= 64) {
      // decode-sized steps: one weight-streaming pass per chosen (token, expert) pair, rows in pair order; identity choices are skipped
      LinearArgs up = linear_args(h, dt, w.e_gu, dt, egu, dt, T * s.top, 2 * s.ff, W);
      up.wbs = gu_stride;
      PickedRows pu = {T * s.top, nullptr, s.top, iota, topi};
      pu.group_limit = s.experts;
      KRN("moe_up", linear_picked_rows(up, pu, st));
      KRN("glu", glu_clamped(egu, 2 * s.ff, eact, s.ff, dt, T * s.top, s.ff, s.limit, 1.702f, st));
      LinearArgs dn = linear_args(eact, dt, w.e_down, dt, edown, DT_F32, T * s.top, W, s.ff);
      dn.wbs = down_stride;
      PickedRows pd = {T * s.top, iota, 1, iota, topi};
      pd.group_limit = s.experts;
      KRN("moe_down", linear_picked_rows(dn, pd, st));
      // pair k of token t is row t * top + k: the combine walks them through an identity table
      KRN("moe_combine", moe_combine_identity(edown, DT_F32, iota, topw, topi, s.experts, h, fo, dt, T, s.top, W, st));
      return rc;
    }
    const int cap = (T * s.top + 63) / 64 * 64 + ne * 64;
    KRN("moe_align", moe_align(topi, T, s.top, ne, sorted_rows, tile_group, pair_pos, cap, st, per_expert ? expert_rows : nullptr, nullptr, nullptr, s.experts));
    if (per_expert) {
      // Large steps: every expert's rows are one tcgen05 GEMM.  The row counts come back to the host (one small copy and a
      // wait per layer, paid only by steps of hundreds of tokens); the inputs are gathered into sorted order.
      KRN("moe_gather", moe_gather_bf16(h, sorted_rows, hsorted, cap, W, st, nullptr));
      if (cudaMemcpyAsync(expert_rows_host, expert_rows, static_cast<size_t>(ne) * 2 * sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
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
      const int real_rows = expert_rows_host[2 * (s.experts - 1)] + (expert_rows_host[2 * (s.experts - 1) + 1] + 63) / 64 * 64;   // rows of experts with matrices
      KRN("glu", glu_clamped(egu, 2 * s.ff, eact, s.ff, dt, real_rows, s.ff, s.limit, 1.702f, st));
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
      KRN("moe_combine", moe_combine_identity(edown16, DT_BF16, pair_pos, topw, topi, s.experts, h, fo, dt, T, s.top, W, st));
      return rc;
    }
    LinearArgs up = linear_args(h, dt, w.e_gu, dt, egu, dt, cap, 2 * s.ff, W);
    up.x_rows = sorted_rows; up.tile_group = tile_group; up.wbs = gu_stride;
    KRN("moe_up", linear(up, st));
    KRN("glu", glu_clamped(egu, 2 * s.ff, eact, s.ff, dt, cap, s.ff, s.limit, 1.702f, st));
    LinearArgs dn = linear_args(eact, dt, w.e_down, dt, edown, DT_F32, cap, W, s.ff);
    dn.tile_group = tile_group; dn.wbs = down_stride;
    KRN("moe_down", linear(dn, st));
    KRN("moe_combine", moe_combine_identity(edown, DT_F32, pair_pos, topw, topi, s.experts, h, fo, dt, T, s.top, W, st));
    return rc;
  }

  int forward(const StepBatch& b, int* sampled, float* host_logits, int64_t* launches) override {
    cudaStream_t st = env.stream;
    const int T = b.T;
    int rc = 0;
    int64_t nl = 0;
    const size_t es = dtype_bytes(dt);
    auto col = [&](void* base, size_t off) { return static_cast<void*>(static_cast<uint8_t*>(base) + off * es); };
    KRN("embed", embed_learned_pos(embed, pos_table, dt, b.ids, b.pos, x, T, W, V, max_pos, ns, xstride, st));
    Pending pend;
    for (size_t li = 0; li < spec.size() && !rc; ++li) {
      const LayerSpec& s = spec[li];
      const LayerWeights& w = wts[li];
      const LayerRun& r = run[li];
      KRN("stream_norm", hyper_step(boundary(pend, w.hc1.in, w.norm1, h, dt, nullptr, T), st));
      KRN("proj_in", project(w.p_in, w.tc_in, xm_h, h, w.w_in, inb, T, s.n_in, W));
      if (s.kind == MIX_PARALLEL) {
        rc |= mix_parallel(s, w, r, b, nl);
        pend.y = ysum; pend.ty = DT_F32;
      } else {
        rc |= mix_mamba(s, w, r, b, nl);
        pend.y = al; pend.ty = dt;
      }
      pend.hc = hyper ? &w.hc1 : nullptr;
      pend.gate = gated ? col(inb, s.off_gate) : nullptr; pend.ldg = s.n_in; pend.gate_bias = w.rg1_b;
      if (s.mlp) {
        KRN("stream_norm", hyper_step(boundary(pend, w.hc2.in, w.norm2, h, dt, nullptr, T), st));
        if (gated) KRN("proj_gate", project(w.p_rg2, w.tc_rg2, xm_h, h, w.rg2, g2, T, W, W));
        rc |= moe(s, w, T, nl);
        pend.y = fo; pend.ty = dt; pend.hc = hyper ? &w.hc2 : nullptr;
        pend.gate = gated ? g2 : nullptr; pend.ldg = W; pend.gate_bias = w.rg2_b;
      }
      if (residual_sink && !rc) {
        // debug: apply the write-back now and read the sum of the streams
        if (!sumbuf && dalloc(&sumbuf, static_cast<size_t>(env.Tcap) * W * sizeof(float))) rc = -3;
        KRN("stream_norm", hyper_step(boundary(pend, nullptr, nullptr, sumbuf, DT_F32, nullptr, T), st));
        pend = Pending();
        const size_t at = residual_sink->size();
        residual_sink->resize(at + static_cast<size_t>(T) * W);
        if (rc || cudaMemcpyAsync(residual_sink->data() + at, sumbuf, static_cast<size_t>(T) * W * sizeof(float), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
            cudaStreamSynchronize(st) != cudaSuccess) rc = -2;
      }
    }
    if (pend.y) KRN("stream_norm", hyper_step(boundary(pend, nullptr, nullptr, nullptr, dt, nullptr, T), st));
    // head: the last norm over the summed streams of the wanted rows (its number carries the logit scale), logits in fp32, greedy choice
    for (int r0 = 0; r0 < b.S && !rc; r0 += row_cap) {
      const int n = std::min(row_cap, b.S - r0);
      KRN("stream_norm", hyper_step(boundary(Pending(), nullptr, fin_w, hrow, dt, b.rows + r0, n), st));
      KRN("head", linear(linear_args(hrow, dt, head, dt, logits, DT_F32, n, V, W), st));
      KRN("argmax", argmax_f32(logits, sampled + r0, n, V, st));
      if (host_logits && cudaMemcpyAsync(host_logits + static_cast<size_t>(r0) * V, logits, static_cast<size_t>(n) * V * sizeof(float),
                                         cudaMemcpyDeviceToHost, st) != cudaSuccess) rc = -2;
    }
    if (launches) *launches += nl;
    if (rc) { set_error("Nagilix forward: %s failed with %d (%s)", failed_kernel, failed_rc, cudaGetErrorString(cudaGetLastError())); return -2; }
    return 0;
  }
};

}  // namespace

#undef KRN

std::unique_ptr<Model> make_nagilix(const JVal& config, DType dtype, std::string* err) {
  std::unique_ptr<Nagilix> m(new Nagilix(dtype));
  if (!m->parse(config, err)) return nullptr;
  return std::unique_ptr<Model>(m.release());
}

}  // namespace b200
