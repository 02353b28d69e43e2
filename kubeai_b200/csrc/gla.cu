// Gated linear attention (mixers.h GlaArgs): a recurrent mixer whose per-head state S [dim, vdim] is decayed per key
// channel and updated with an outer product, S_t = diag(alpha_t) S_{t-1} + k_t v_t^T, o_t = S_t^T q_t.
//
// The scan is sequential in the token and exact: the same fp32 operations in the same order whether a sequence's tokens
// arrive in one step or one at a time, so chunked prefill and decode agree bit for bit.  Parallelism comes from the
// independent columns of S: a thread owns one or two value columns j and a slice of the key rows, and keeps that slice of
// the state in registers for the whole step.  The P = 1, 2, 4 ... row slices of a column live in different warps (a warp
// reads one slice of q, k and the decay as a shared-memory broadcast); their partial outputs meet in shared memory and are
// added in a fixed order.  The decay alpha = exp(inv_tau * logsigmoid(z + bias)) is computed once per step by its own
// elementwise kernel, in fp32 with the accurate library functions; q, k and alpha of a group of tokens are staged in
// shared memory once per CTA.  The state lives in HBM between steps ([slot][head][dim][vdim] fp32) and is read and
// written once per step.
//
// The same scan serves recurrences whose gates are scalars per (token, head) (tok_decay / tok_kscale), among them the
// matrix memory with exponential gating (mLSTM): its gates come from `mlstm_gates`, its normaliser n_t = d n + s k and the
// product n . q ride along in the scan's first column block (GlaArgs::nstate / nq), and `recurrent_out_gate` divides by
// max(|n . q|, exp(-m)) before the norm.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <stdlib.h>

#include <algorithm>

#include "mixers.h"

namespace b200 {
namespace {

typedef __nv_bfloat16 bf16;
__device__ __forceinline__ float ldf(const float* p) { return __ldg(p); }
__device__ __forceinline__ float ldf(const bf16* p) { return __bfloat162float(__ldg(p)); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(bf16* p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ float siluf_(float x) { return x / (1.0f + expf(-x)); }

constexpr int kRows = 32;      // key rows of the state held by one thread
constexpr int kGroup = 16;     // tokens staged per shared-memory round (fewer when dim is large)
constexpr int kThreads = 128;

// grid: (ceil(vdim / (kThreads / P)), heads, nseq); P = row slices per column (a power of two), rpp = key rows per slice
// (a multiple of 4, P * rpp >= dim, rpp <= kRows).  G tokens are staged per round: q (scaled), k, alpha as [G][3][P][rpp + 4]
// (rows past dim are zeros; the 4-float pad puts the P slices a thread group reads at once into different banks, and a
// thread reads its slice as float4), then v and o for the CTA's columns [G][cols] each, so the sequential token loop
// touches shared memory only.
// The decay of every (token, head, key channel), once per step and in place over the pre-activation:
// alpha = exp(inv_tau * logsigmoid(z + bias)), log sigmoid(z) = min(z, 0) - log1p(exp(-|z|)), accurate fp32 functions.
__global__ void gla_decay_kernel(float* z, const float* bias, int HD, float inv_tau, long long total) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const float v = z[i] + bias[i % HD];
  const float ls = fminf(v, 0.f) - log1pf(expf(-fabsf(v)));
  z[i] = expf(ls * inv_tau);
}

// NC = value columns per thread (2 when the value width keeps every SM busy with half as many CTAs: each q, k, alpha read
// from shared memory then feeds twice the arithmetic).  Threads of a warp share one row slice (part = thread / tcols), so a
// shared-memory read of q, k or alpha is one broadcast; the P partial outputs of a column meet in shared memory and are
// summed by the pass that writes the round's outputs.
// MODE 0: learned per-channel decays, staged as a third row.  MODE 1: one constant decay per head (GlaArgs::head_decay): no
// decay row is staged or read, the constant sits in a register.  MODE 2: one decay and one key scale per (token, head)
// (GlaArgs::tok_decay / tok_kscale): both sit in shared memory as G scalars per round; the key scale multiplies the token's
// value (and the normaliser's key) in the chain, (s k) v^T = k (s v)^T.
// NRM (with MODE 2): the CTAs of the first column block also carry the normaliser n [dim] of the head, n <- decay n + k
// (what the scan does to a state column whose value is 1).  The threads of a row slice share its rows (thread jj owns rows
// jj, jj + tcols, ... of the slice, at most kNormRows of them); every thread leaves its part of n . q in shared memory, and
// the pass that writes the round's outputs sums the parts in a fixed order.
// NE = rows of n per thread: 1 covers dim <= 128 (a slice has no more rows than threads), kNormRows the rest; 0 = no normaliser.
constexpr int kNormRows = 8;
template <typename T, int NC, int MODE, int NE>
__global__ void __launch_bounds__(kThreads) gla_scan_kernel(GlaArgs a, int P, int rpp, int G) {
  constexpr bool CD = MODE != 0;
  constexpr bool NRM = NE > 0;
  extern __shared__ __align__(16) float sm[];
  const int seq = blockIdx.z, head = blockIdx.y;
  const int tok0 = a.seqs[seq * 8 + 0], n = a.seqs[seq * 8 + 1], pos0 = a.seqs[seq * 8 + 2], slot = a.seqs[seq * 8 + 3];
  const int D = a.dim, Dv = a.vdim;
  const int tcols = kThreads / P, cols = tcols * NC;   // columns per thread group, per CTA
  const int part = threadIdx.x / tcols, jj = threadIdx.x % tcols;
  int j[NC];
  bool live[NC];
#pragma unroll
  for (int c = 0; c < NC; ++c) { j[c] = blockIdx.x * cols + jj + c * tcols; live[c] = j[c] < Dv; }
  const int i0 = part * rpp;
  const int ps = rpp + 4, Dp = P * ps;     // padded slice and row length
  float* vs = sm + static_cast<size_t>(G) * 3 * Dp;   // [G][cols]
  float* os = vs + G * cols;                          // [G][P][cols]
  float* ds = os + G * P * cols;                      // [2][G] the round's decays and key scales (MODE 2)
  // behind the decays: [G][threads] partial n . q (NRM)
  const bool nrm = NRM && blockIdx.x == 0;
  float nv[NRM ? NE : 1];
  if (NRM) {
    const float* nst = a.nstate + (static_cast<long long>(slot) * a.heads + head) * D;
#pragma unroll
    for (int e = 0; e < NE; ++e) {
      const int r = jj + e * tcols, i = i0 + r;
      nv[e] = (nrm && r < rpp && i < D && pos0 > 0) ? nst[i] : 0.f;
    }
  }
  const T* base = static_cast<const T*>(a.qkv);
  float* Sg = a.states + ((static_cast<long long>(slot) * a.heads + head) * D) * Dv;
  float S[NC][kRows];
#pragma unroll
  for (int c = 0; c < NC; ++c)
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      const int i = i0 + r;
      S[c][r] = (live[c] && r < rpp && i < D && pos0 > 0) ? Sg[static_cast<long long>(i) * Dv + j[c]] : 0.f;
    }
  const int slice_elems = P * rpp;
  const bool silu = a.act == GLA_ACT_SILU;
  const float hdecay = MODE == 1 ? a.head_decay[head] : 0.f;
  for (int g0 = 0; g0 < n; g0 += G) {
    const int gn = min(G, n - g0);
    __syncthreads();
    // stage q (scaled), k, alpha of the round's tokens: element x of a token's padded row belongs to slice x / rpp
    for (int x = threadIdx.x; x < slice_elems; x += kThreads) {
      const int pp = x / rpp, r = x - pp * rpp, i = pp * rpp + r;
      float* s3 = sm + pp * ps + r;
      const int c = head * D + i;
      if (i < D) {
#pragma unroll 4
        for (int tt = 0; tt < gn; ++tt) {
          const long long row = static_cast<long long>(tok0 + g0 + tt);
          const T* rp = base + row * a.ld;
          float qv = ldf(rp + a.q_off + c), kv = ldf(rp + a.k_off + c);
          if (silu) { qv = siluf_(qv); kv = siluf_(kv); }
          if (a.rope && i < a.rot_dims) {
            // rotate-half layout: dimension i of the head is paired with i + rot_dims / 2
            const int half = a.rot_dims >> 1;
            const bool low = i < half;
            const int cp = low ? c + half : c - half;
            const float2 r = __ldg(a.rope + static_cast<long long>(pos0 + g0 + tt) * half + (low ? i : i - half));
            const float qo = ldf(rp + a.q_off + cp), ko = ldf(rp + a.k_off + cp);
            qv = low ? qv * r.x - qo * r.y : qv * r.x + qo * r.y;
            kv = low ? kv * r.x - ko * r.y : kv * r.x + ko * r.y;
          }
          s3[(tt * 3) * Dp] = qv * a.q_scale;
          s3[(tt * 3 + 1) * Dp] = kv * a.k_scale;
          if (!CD) s3[(tt * 3 + 2) * Dp] = __ldg(a.z + row * (a.heads * D) + c);
        }
      } else {
        for (int tt = 0; tt < gn; ++tt) { s3[(tt * 3) * Dp] = 0.f; s3[(tt * 3 + 1) * Dp] = 0.f; s3[(tt * 3 + 2) * Dp] = 0.f; }
      }
    }
    for (int e = threadIdx.x; e < gn * cols; e += kThreads) {
      const int tt = e / cols, c = e - tt * cols, jc = blockIdx.x * cols + c;
      float vv = jc < Dv ? ldf(base + static_cast<long long>(tok0 + g0 + tt) * a.ld + a.v_off + head * Dv + jc) : 0.f;
      if (silu) vv = siluf_(vv);
      vs[e] = vv;
    }
    if (MODE == 2)
      for (int tt = threadIdx.x; tt < gn; tt += kThreads) {
        ds[tt] = __ldg(a.tok_decay + static_cast<long long>(tok0 + g0 + tt) * a.heads + head);
        ds[G + tt] = __ldg(a.tok_kscale + static_cast<long long>(tok0 + g0 + tt) * a.heads + head);
      }
    __syncthreads();
    for (int tt = 0; tt < gn; ++tt) {
      const float decay = MODE == 2 ? ds[tt] : hdecay;
      const float kscale = MODE == 2 ? ds[G + tt] : 1.f;   // the key's scalar gate multiplies the value instead: (s k) v = k (s v)
      float v[NC], o[NC][4];
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        v[c] = vs[tt * cols + jj + c * tcols];
        if (MODE == 2) v[c] *= kscale;
        o[c][0] = o[c][1] = o[c][2] = o[c][3] = 0.f;
      }
      const float4* q4 = reinterpret_cast<const float4*>(sm + (tt * 3) * Dp + part * ps);
      const float4* k4 = reinterpret_cast<const float4*>(sm + (tt * 3 + 1) * Dp + part * ps);
      const float4* a4 = reinterpret_cast<const float4*>(sm + (tt * 3 + 2) * Dp + part * ps);
#pragma unroll
      for (int m = 0; m < kRows / 4; ++m) {
        if (4 * m < rpp) {
          const float4 qa = q4[m], ka = k4[m], aa = CD ? make_float4(decay, decay, decay, decay) : a4[m];
#pragma unroll
          for (int c = 0; c < NC; ++c) {
            float* Sc = S[c] + 4 * m;
            Sc[0] = fmaf(aa.x, Sc[0], ka.x * v[c]); o[c][0] = fmaf(Sc[0], qa.x, o[c][0]);
            Sc[1] = fmaf(aa.y, Sc[1], ka.y * v[c]); o[c][1] = fmaf(Sc[1], qa.y, o[c][1]);
            Sc[2] = fmaf(aa.z, Sc[2], ka.z * v[c]); o[c][2] = fmaf(Sc[2], qa.z, o[c][2]);
            Sc[3] = fmaf(aa.w, Sc[3], ka.w * v[c]); o[c][3] = fmaf(Sc[3], qa.w, o[c][3]);
          }
        }
      }
#pragma unroll
      for (int c = 0; c < NC; ++c) os[(tt * P + part) * cols + jj + c * tcols] = (o[c][0] + o[c][1]) + (o[c][2] + o[c][3]);
      if (NRM && nrm) {
        const float* qs = reinterpret_cast<const float*>(q4);
        const float* ks = reinterpret_cast<const float*>(k4);
        float nacc = 0.f;
#pragma unroll
        for (int e = 0; e < NE; ++e) {
          const int r = jj + e * tcols;
          if (r < rpp) {
            nv[e] = fmaf(decay, nv[e], ks[r] * kscale);
            nacc = fmaf(nv[e], qs[r], nacc);
          }
        }
        (os + G * P * cols + 2 * G)[tt * kThreads + threadIdx.x] = nacc;   // summed over the threads by the output pass: no reduction inside the token chain
      }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < gn * cols; e += kThreads) {
      const int tt = e / cols, c = e - tt * cols, jc = blockIdx.x * cols + c;
      float o = 0.f;
      for (int pp = 0; pp < P; ++pp) o += os[(tt * P + pp) * cols + c];   // slices in a fixed order
      if (jc < Dv) a.o[static_cast<long long>(tok0 + g0 + tt) * (a.heads * Dv) + head * Dv + jc] = o;
    }
    if (NRM && nrm)
      for (int tt = threadIdx.x >> 5; tt < gn; tt += kThreads / 32) {   // a warp per token: the threads' partial products in a fixed order
        const int lane = threadIdx.x & 31;
        const float* pq = ds + 2 * G + tt * kThreads;
        float q = (pq[lane] + pq[lane + 32]) + (pq[lane + 64] + pq[lane + 96]);
        for (int sft = 16; sft > 0; sft >>= 1) q += __shfl_xor_sync(0xffffffffu, q, sft);
        if (lane == 0) a.nq[static_cast<long long>(tok0 + g0 + tt) * a.heads + head] = q;
      }
  }
  if (NRM && nrm) {
    float* nst = a.nstate + (static_cast<long long>(slot) * a.heads + head) * D;
#pragma unroll
    for (int e = 0; e < NE; ++e) {
      const int r = jj + e * tcols, i = i0 + r;
      if (r < rpp && i < D) nst[i] = nv[e];
    }
  }
#pragma unroll
  for (int c = 0; c < NC; ++c)
    if (live[c]) {
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        const int i = i0 + r;
        if (r < rpp && i < D) Sg[static_cast<long long>(i) * Dv + j[c]] = S[c][r];
      }
    }
}

// one warp per (token, head): unit RMS over vdim, weight, SiLU gate
template <typename T>
__global__ void gla_out_gate_kernel(const float* o, const T* g, int ldg, const float* w, float eps, T* y, int ldy, int heads, int vdim, long long pairs) {
  const long long p = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (p >= pairs) return;
  const int lane = threadIdx.x & 31;
  const long long t = p / heads;
  const int h = static_cast<int>(p - t * heads);
  const float* op = o + p * vdim;
  float ss = 0.f;
  for (int i = lane; i < vdim; i += 32) ss = fmaf(op[i], op[i], ss);
  for (int s = 16; s > 0; s >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, s);
  const float inv = 1.0f / sqrtf(ss / static_cast<float>(vdim) + eps);
  for (int i = lane; i < vdim; i += 32) {
    const float gv = ldf(g + t * ldg + h * vdim + i);
    stf(y + t * ldy + h * vdim + i, op[i] * inv * w[i] * (gv / (1.0f + expf(-gv))));
  }
}

// The general output stage.  Per-head norm: one warp per (token, head).  Norm over the concatenated heads: one CTA per
// token, the warps' sums of squares added in warp order.
template <typename T>
__global__ void recurrent_out_gate_kernel(OutGateArgs a, long long units) {
  __shared__ float red[8];
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5;
  long long t;
  int c0, n, first, step;
  if (a.joint) {
    t = blockIdx.x; c0 = 0; n = a.heads * a.vdim; first = threadIdx.x; step = blockDim.x;
  } else {
    const long long p = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + wrp;
    if (p >= units) return;
    t = p / a.heads; c0 = static_cast<int>(p - t * a.heads) * a.vdim; n = a.vdim; first = lane; step = 32;
  }
  const float* op = a.o + t * (static_cast<long long>(a.heads) * a.vdim) + c0;
  // a normalised recurrence: the head's outputs are divided by max(|n . q|, floor) + den_eps before the norm
  const long long th = t * a.heads + c0 / a.vdim;
  const float dinv = a.den_nq ? 1.0f / (fmaxf(fabsf(a.den_nq[th]), a.den_floor[th]) + a.den_eps) : 1.0f;
  const float* w = a.w ? a.w + (a.w_full ? c0 : 0) : nullptr;   // null: a norm without a weight
  const T* g = static_cast<const T*>(a.g) + t * a.ldg + c0;
  T* y = static_cast<T*>(a.y) + t * a.ldy + c0;
  float ss = 0.f;
  for (int i = first; i < n; i += step) { const float v = op[i] * dinv; ss = fmaf(v, v, ss); }
  for (int s = 16; s > 0; s >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, s);
  if (a.joint) {
    if (lane == 0) red[wrp] = ss;
    __syncthreads();
    ss = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) ss += red[w];
  }
  const float inv = 1.0f / sqrtf(ss / static_cast<float>(n) + a.eps);
  for (int i = first; i < n; i += step) {
    const float gv = ldf(g + i);
    const float sg = 1.0f / (1.0f + expf(-gv));
    const float gate = a.gate_act == GATE_SIGMOID ? sg : gv * sg;
    stf(y + i, op[i] * dinv * inv * (w ? w[i] : 1.0f) * gate * a.out_scale);
  }
}

// The scalar gates of the matrix-memory recurrence (MlstmGateArgs).  One CTA per (head, sequence) walks the sequence's
// tokens in rounds: all threads turn a round's pre-activations into the log gates (accurate tanhf, log1pf, expf), ONE
// thread runs the chain m_t = max(f_t + m_(t-1), i_t) over the round from shared memory (an add and a max per token,
// the same operations in the same order however the sequence was cut into steps), all threads turn (i, f, m) into the
// three factors the scan and the output stage read.
constexpr int kGateRound = 512;
__global__ void __launch_bounds__(128) mlstm_gates_kernel(MlstmGateArgs a) {
  __shared__ float li[kGateRound], lf[kGateRound], ms[kGateRound + 1];
  const int head = blockIdx.x, seq = blockIdx.y;
  const int tok0 = a.seqs[seq * 8 + 0], n = a.seqs[seq * 8 + 1], pos0 = a.seqs[seq * 8 + 2], slot = a.seqs[seq * 8 + 3];
  float* mst = a.mstate + static_cast<long long>(slot) * a.heads + head;
  if (threadIdx.x == 0) ms[0] = pos0 > 0 ? *mst : 0.f;
  for (int g0 = 0; g0 < n; g0 += kGateRound) {
    const int gn = min(kGateRound, n - g0);
    for (int tt = threadIdx.x; tt < gn; tt += blockDim.x) {
      const float* row = a.pre + static_cast<long long>(tok0 + g0 + tt) * a.ld;
      float zi = row[head], zf = row[a.heads + head];
      if (a.cap > 0.f) { zi = a.cap * tanhf(zi / a.cap); zf = a.cap * tanhf(zf / a.cap); }
      li[tt] = zi;
      lf[tt] = fminf(zf, 0.f) - log1pf(expf(-fabsf(zf)));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float m = ms[0];
      for (int tt = 0; tt < gn; ++tt) { m = fmaxf(lf[tt] + m, li[tt]); ms[tt + 1] = m; }
    }
    __syncthreads();
    for (int tt = threadIdx.x; tt < gn; tt += blockDim.x) {
      const long long o = static_cast<long long>(tok0 + g0 + tt) * a.heads + head;
      const float mp = ms[tt], mn = ms[tt + 1];
      a.keep[o] = expf(lf[tt] + mp - mn);
      a.take[o] = expf(li[tt] - mn);
      a.floor[o] = expf(-mn);
    }
    __syncthreads();
    if (threadIdx.x == 0) ms[0] = ms[gn];
  }
  __syncthreads();
  if (threadIdx.x == 0 && n > 0) *mst = ms[0];
}

}  // namespace

int mlstm_gates(const MlstmGateArgs& a, cudaStream_t st) {
  if (a.nseq <= 0) return 0;
  if (!a.pre || !a.keep || !a.take || !a.floor || !a.mstate || !a.seqs || a.heads < 1 || a.ld < 2 * a.heads) return -1;
  mlstm_gates_kernel<<<dim3(a.heads, a.nseq), 128, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int recurrent_out_gate(const OutGateArgs& a, cudaStream_t st) {
  const long long units = a.joint ? a.T : static_cast<long long>(a.T) * a.heads;
  if (units <= 0) return 0;
  if (!a.o || !a.g || !a.y || a.heads < 1 || a.vdim < 1) return -1;
  if (a.joint && (a.w_full || a.den_nq)) return -1;
  if (a.den_nq && !a.den_floor) return -1;
  const int th = a.joint ? (a.heads * a.vdim >= 1024 ? 256 : 128) : 128;
  const unsigned grid = static_cast<unsigned>(a.joint ? units : (units + 3) / 4);
  if (a.t == DT_BF16) recurrent_out_gate_kernel<bf16><<<grid, th, 0, st>>>(a, units);
  else recurrent_out_gate_kernel<float><<<grid, th, 0, st>>>(a, units);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int gla_scan(const GlaArgs& a, cudaStream_t st) {
  if (a.nseq <= 0) return 0;
  if (a.dim < 1 || a.vdim < 1 || a.heads < 1) return -1;
  if (a.rope && (a.rot_dims < 2 || a.rot_dims % 2 || a.rot_dims > a.dim || a.act != GLA_ACT_NONE)) return -1;
  int P = 1;
  while (P * kRows < a.dim) P <<= 1;
  if (P > 32) return -1;   // dim <= 1024
  const int rows_per_part = ((a.dim + P - 1) / P + 3) / 4 * 4;
  const int tcols = kThreads / P;
  // two columns per thread when that still leaves at least two CTAs per SM's worth of work
  int sms = 148;
  { int dev = 0; if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
  const long long ctas2 = static_cast<long long>((a.vdim + 2 * tcols - 1) / (2 * tcols)) * a.heads * a.nseq;
  int NC = (a.vdim >= 2 * tcols && ctas2 >= sms) ? 2 : 1;
  if (const char* e = getenv("B200_GLA_NC")) NC = atoi(e) == 2 && a.vdim >= 2 * tcols ? 2 : 1;   // A/B knob
  const int cols = tcols * NC;
  dim3 grid((a.vdim + cols - 1) / cols, a.heads, a.nseq);
  int G = kGroup;
  if (const char* e = getenv("B200_GLA_GROUP")) G = std::max(1, atoi(e));   // A/B knob: tokens staged per round
  auto smem_for = [&](int g) { return static_cast<size_t>(g) * (3 * P * (rows_per_part + 4) + (1 + P) * cols + 2 + (a.nstate ? kThreads : 0)) * sizeof(float); };
  while (G > 1 && smem_for(G) > 44 * 1024) G >>= 1;
  const size_t smem = smem_for(G);
  if (smem > 48 * 1024) return -1;
  if ((a.nstate != nullptr) != (a.nq != nullptr) || (a.nstate && !a.tok_decay)) return -1;
  if (a.nstate && rows_per_part > kNormRows * tcols) return -1;
  if (a.tok_decay) {
    if (!a.tok_kscale || a.head_decay) return -1;
  } else if (!a.head_decay) {
    if (!a.z || !a.z_bias) return -1;
    const long long total = static_cast<long long>(a.T) * a.heads * a.dim;
    if (total > 0) gla_decay_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, st>>>(a.z, a.z_bias, a.heads * a.dim, a.inv_tau, total);
  }
  const bool one_row = rows_per_part <= tcols;
#define SCAN(T_, NC_) do { if (a.tok_decay && a.nstate && one_row) gla_scan_kernel<T_, NC_, 2, 1><<<grid, kThreads, smem, st>>>(a, P, rows_per_part, G); \
                          else if (a.tok_decay && a.nstate) gla_scan_kernel<T_, NC_, 2, kNormRows><<<grid, kThreads, smem, st>>>(a, P, rows_per_part, G); \
                          else if (a.tok_decay) gla_scan_kernel<T_, NC_, 2, 0><<<grid, kThreads, smem, st>>>(a, P, rows_per_part, G); \
                          else if (a.head_decay) gla_scan_kernel<T_, NC_, 1, 0><<<grid, kThreads, smem, st>>>(a, P, rows_per_part, G); \
                          else gla_scan_kernel<T_, NC_, 0, 0><<<grid, kThreads, smem, st>>>(a, P, rows_per_part, G); } while (0)
  if (a.t == DT_BF16) {
    if (NC == 2) SCAN(bf16, 2); else SCAN(bf16, 1);
  } else {
    if (NC == 2) SCAN(float, 2); else SCAN(float, 1);
  }
#undef SCAN
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int gla_out_gate(const float* o, const void* g, int ldg, const float* w, float eps, void* y, int ldy, DType t, int T, int heads, int vdim, cudaStream_t st) {
  const long long pairs = static_cast<long long>(T) * heads;
  if (pairs <= 0) return 0;
  const unsigned grid = static_cast<unsigned>((pairs + 3) / 4);
  if (t == DT_BF16) gla_out_gate_kernel<bf16><<<grid, 128, 0, st>>>(o, static_cast<const bf16*>(g), ldg, w, eps, static_cast<bf16*>(y), ldy, heads, vdim, pairs);
  else gla_out_gate_kernel<float><<<grid, 128, 0, st>>>(o, static_cast<const float*>(g), ldg, w, eps, static_cast<float*>(y), ldy, heads, vdim, pairs);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // namespace b200
