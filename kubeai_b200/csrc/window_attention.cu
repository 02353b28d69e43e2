// Softmax attention with grouped key/value heads over a paged cache, a sliding window and kept first tokens
// (mixers.h WindowAttnArgs), with the preparation in front of it: interleaved rotary positions under YaRN-style
// frequency scaling and a unit-RMS norm of every query and key head, optionally with a weight, a position-dependent query
// gain and a blend of the values with an earlier layer's (QkPrepArgs).  Scores may be tanh-capped, the sigmoid output
// gate is per output column or per head.  A second preparation (ConvQkPrepArgs) serves attention whose queries and keys
// pass a short causal convolution, a norm over the whole projection and a rotate-half rotation, and whose values are the
// convolved keys.  Visibility may be chunked instead of windowed (the first visible key is the start of the token's
// chunk), and the softmax may have a sink, a learned per-head term exp(sink) of the denominator that belongs to no cached token.
//
// Visibility of key j for the token at position p: j <= p and (p - j < window or j < keep_first).  The visible keys of
// a token are therefore two runs, [0, min(keep_first, lo)) and [lo, p] with lo = max(0, p - window + 1); both kernels
// walk exactly those and nothing else, in an order that depends only on p, so the result does not depend on how a
// prompt was cut into steps or on what shares the batch.  Kept tokens keep their own positions: keys are rotated once,
// when they are written, and never again.
//
// Kernels: `qk_prep_kernel` (one CTA per token: rotate, normalise, write the cache row), `window_attn_kernel` (any head
// size, bf16 or fp32 cache: one CTA per (token, head), its warps share the token's keys in 32-key chunks, a lane owns
// one key for the scores and a slice of the value columns for the output, online softmax in fp32, the warps' partial
// results meet in shared memory in a fixed order; the sigmoid output gate and the branch scale are applied before the
// single rounding to the storage type), and `window_attn_mma_kernel` (bf16, head sizes that fit the mma.sync fragments:
// 64 query rows of one sequence, the heads of one key/value group together, against 64-key tiles on the tensor cores).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <math.h>
#include <stdlib.h>

#include <algorithm>
#include <vector>

#include "launch.h"
#include "mixers.h"

namespace b200 {
namespace {

typedef __nv_bfloat16 bf16;
__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const bf16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(bf16* p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }

// ---------------------------------------------------------------------------------------------- rotation, norm, cache write
// One CTA per token; a warp takes the heads u = warp, warp + nwarps, ...: u < heads is a query head, the next kv_heads are
// key heads.  A lane owns the dimension pairs (2i, 2i + 1), i = lane, lane + 32, ...; the odd last dimension of an odd dim is
// lane 0's.  Value rows are copied by all threads.
template <typename T>
__global__ void __launch_bounds__(128) qk_prep_kernel(QkPrepArgs a) {
  const long long t = blockIdx.x;
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int p = a.positions[t];
  const long long slot = a.slots[t];
  const int D = a.dim, half = a.rot_dims / 2, pairs = D / 2;
  const float2* cs = half ? a.rope + static_cast<long long>(p) * half : nullptr;
  // the query gain of this position: 1 + coef ln(floor((p + 1) / every) + 1), in fp32 with the accurate logarithm
  const float q_gain = a.q_gain_every > 0 ? 1.0f + a.q_gain_coef * logf(static_cast<float>((p + 1) / a.q_gain_every + 1)) : 1.0f;
  const long long crow = static_cast<long long>(a.kv_heads) * (D + a.vdim);
  T* cache = static_cast<T*>(a.cache) + slot * crow;
  for (int u = wrp; u < a.heads + a.kv_heads; u += nw) {
    const bool isq = u < a.heads;
    const T* src = isq ? static_cast<const T*>(a.q) + t * a.ld + static_cast<long long>(u) * D
                       : static_cast<const T*>(a.k) + t * a.ld + static_cast<long long>(u - a.heads) * D;
    // rotate, accumulate the sum of squares; the rotated values are recomputed in the second pass (cheaper than a spill)
    float ss = 0.f;
    for (int i = lane; i < pairs; i += 32) {
      float x0 = ldf(src + 2 * i), x1 = ldf(src + 2 * i + 1);
      if (i < half) {
        const float2 c = cs[i];
        const float r0 = x0 * c.x - x1 * c.y, r1 = x1 * c.x + x0 * c.y;
        x0 = r0; x1 = r1;
      }
      ss = fmaf(x0, x0, ss);
      ss = fmaf(x1, x1, ss);
    }
    if ((D & 1) && lane == 0) { const float x = ldf(src + D - 1); ss = fmaf(x, x, ss); }
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = (a.unit_norm ? 1.0f / sqrtf(ss / static_cast<float>(D) + a.eps) : 1.0f) * (isq ? q_gain : 1.0f);
    const float* nw = isq ? a.q_norm_w : a.k_norm_w;   // optional weight of the norm, shared by the heads
    for (int i = lane; i < pairs; i += 32) {
      float x0 = ldf(src + 2 * i), x1 = ldf(src + 2 * i + 1);
      if (i < half) {
        const float2 c = cs[i];
        const float r0 = x0 * c.x - x1 * c.y, r1 = x1 * c.x + x0 * c.y;
        x0 = r0; x1 = r1;
      }
      x0 *= inv; x1 *= inv;
      if (nw) { x0 *= nw[2 * i]; x1 *= nw[2 * i + 1]; }
      if (isq) {
        float* dst = a.qn + (t * a.heads + u) * D;
        dst[2 * i] = x0; dst[2 * i + 1] = x1;
      } else {
        T* dst = cache + static_cast<long long>(u - a.heads) * D;
        stf(dst + 2 * i, x0); stf(dst + 2 * i + 1, x1);
      }
    }
    if ((D & 1) && lane == 0) {
      const float x = ldf(src + D - 1) * inv * (nw ? nw[D - 1] : 1.0f);
      if (isq) a.qn[(t * a.heads + u) * D + D - 1] = x;
      else stf(cache + static_cast<long long>(u - a.heads) * D + D - 1, x);
    }
  }
  const T* v = static_cast<const T*>(a.v) + t * a.ld;
  T* vdst = cache + static_cast<long long>(a.kv_heads) * D;
  const T* vb = a.v_blend ? static_cast<const T*>(a.v_blend) + t * a.ld_blend : nullptr;
  T* vraw = a.v_raw_out ? static_cast<T*>(a.v_raw_out) + t * a.ld_raw : nullptr;
  for (int i = threadIdx.x; i < a.kv_heads * a.vdim; i += blockDim.x) {
    const T vi = v[i];
    if (vraw) vraw[i] = vi;
    if (vb) stf(vdst + i, (1.0f - a.v_lambda) * ldf(&vi) + a.v_lambda * ldf(vb + i));
    else vdst[i] = vi;
  }
}

// ---------------------------------------------------------------------------------------------- convolved queries and keys
// One CTA per token (ConvQkPrepArgs).  Pass 1: a thread per channel convolves the projections over time (its taps come
// from the step's own rows or from the sequence's carried inputs), leaves the result in shared memory, writes the
// convolved keys as the values of the cache row and adds to the sum of squares of the query row or of the key row; the two
// sums meet in shared memory in warp order.  Pass 2: a thread per rotation pair (dimension i with i + rot_dims / 2) or
// unrotated column normalises over the WHOLE projection, applies the weights, rotates, applies the head's temperature to
// queries and writes qn or the key part of the cache row.
template <typename T>
__global__ void __launch_bounds__(1024) conv_qk_prep_kernel(ConvQkPrepArgs a) {
  extern __shared__ float cv[];   // [(heads + kv_heads) * dim] convolved projections
  __shared__ float red[2][32];
  const long long t = blockIdx.x;
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int D = a.dim, HD = a.heads * D, GD = a.kv_heads * D, C = HD + GD;
  const int p = a.positions[t];
  const long long slot = a.slots[t];
  const int* sq = a.seqs + a.seq_of_tok[t] * 8;
  const int i0 = static_cast<int>(t) - sq[0];
  const bool carried = sq[2] > 0;
  const int taps = a.conv_w ? a.taps : 1;
  const float* st = a.conv_state ? a.conv_state + static_cast<long long>(sq[3]) * (taps - 1) * C : nullptr;
  const T* u = static_cast<const T*>(a.qk);
  T* cache = static_cast<T*>(a.cache) + slot * (2ll * GD);
  float ssq = 0.f, ssk = 0.f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc;
    if (a.conv_w) {
      acc = 0.f;
      const float* wc = a.conv_w + static_cast<long long>(c) * taps;
      if (i0 >= taps - 1) {
        // every tap lies in the step's own rows
        const T* up = u + (t - (taps - 1)) * a.ld + c;
        for (int j = 0; j < taps; ++j) acc = fmaf(wc[j], ldf(up + static_cast<long long>(j) * a.ld), acc);
      } else {
        for (int j = 0; j < taps; ++j) {
          const int d = taps - 1 - j;
          float v = 0.f;
          if (i0 - d >= 0) v = ldf(u + (t - d) * a.ld + c);
          else if (carried) v = st[static_cast<long long>(taps - 1 + i0 - d) * C + c];
          acc = fmaf(wc[j], v, acc);
        }
      }
    } else {
      acc = ldf(u + t * a.ld + c);
    }
    cv[c] = acc;
    if (c < HD) ssq = fmaf(acc, acc, ssq);
    else { ssk = fmaf(acc, acc, ssk); stf(cache + GD + (c - HD), acc); }
  }
  for (int o = 16; o > 0; o >>= 1) { ssq += __shfl_xor_sync(0xffffffffu, ssq, o); ssk += __shfl_xor_sync(0xffffffffu, ssk, o); }
  if (lane == 0) { red[0][wrp] = ssq; red[1][wrp] = ssk; }
  __syncthreads();
  float tq = 0.f, tk = 0.f;
  for (int w = 0; w < nw; ++w) { tq += red[0][w]; tk += red[1][w]; }
  const float invq = 1.0f / sqrtf(tq / static_cast<float>(HD) + a.eps), invk = 1.0f / sqrtf(tk / static_cast<float>(GD) + a.eps);
  const int half = a.rot_dims / 2;
  const float2* cs = half ? a.rope + static_cast<long long>(p) * half : nullptr;
  // a thread takes an item of a head: a rotation pair (columns i and i + half, both outputs) or a column past the rotated ones
  const int per_head = D - half, items = (a.heads + a.kv_heads) * per_head;
  for (int it = threadIdx.x; it < items; it += blockDim.x) {
    const int u_ = it / per_head, k = it - u_ * per_head;
    const bool isq = u_ < a.heads;
    const int hd = isq ? u_ : u_ - a.heads;
    const int cc = hd * D + (k < half ? k : k + half);     // column within the query or the key row
    const float inv = isq ? invq : invk;
    const float* nwt = isq ? a.q_norm_w : a.k_norm_w;
    const float* row = cv + (isq ? 0 : HD);
    const float hs = (isq && a.q_head_scale) ? a.q_head_scale[hd] : 1.0f;
    const float lo = row[cc] * inv * (nwt ? nwt[cc] : 1.0f);
    if (k < half) {
      const float hi = row[cc + half] * inv * (nwt ? nwt[cc + half] : 1.0f);
      const float2 r = cs[k];
      const float o0 = lo * r.x - hi * r.y, o1 = hi * r.x + lo * r.y;
      if (isq) { a.qn[t * HD + cc] = o0 * hs; a.qn[t * HD + cc + half] = o1 * hs; }
      else { stf(cache + cc, o0); stf(cache + cc + half, o1); }
    } else {
      if (isq) a.qn[t * HD + cc] = lo * hs;
      else stf(cache + cc, lo);
    }
  }
}

// ---------------------------------------------------------------------------------------------- attention, any head size
constexpr int kWarps = 4, kWarpsDecode = 16;
constexpr int kMaxVR = 8;   // value columns per lane: vdim <= 256

template <typename T>
__device__ __forceinline__ float dot_row(const float* q, const T* k, int D, bool vec) {
  float acc = 0.f;
  if (vec) {
    if constexpr (sizeof(T) == 2) {
      for (int d = 0; d < D; d += 8) {
        const uint4 v = *reinterpret_cast<const uint4*>(k + d);
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc = fmaf(q[d + 2 * i], __uint_as_float(u[i] << 16), acc);
          acc = fmaf(q[d + 2 * i + 1], __uint_as_float(u[i] & 0xffff0000u), acc);
        }
      }
    } else {
      for (int d = 0; d < D; d += 4) {
        const float4 v = *reinterpret_cast<const float4*>(k + d);
        acc = fmaf(q[d], v.x, acc); acc = fmaf(q[d + 1], v.y, acc); acc = fmaf(q[d + 2], v.z, acc); acc = fmaf(q[d + 3], v.w, acc);
      }
    }
  } else {
    for (int d = 0; d < D; ++d) acc = fmaf(q[d], ldf(k + d), acc);
  }
  return acc;
}

template <typename T>
__global__ void __launch_bounds__(kWarpsDecode * 32) window_attn_kernel(WindowAttnArgs a, bool vec) {
  extern __shared__ float sm[];   // q [dim] | per warp: m, l, acc [vdim]
  const long long t = blockIdx.x / a.heads;
  const int h = blockIdx.x % a.heads;
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int D = a.dim, Dv = a.vdim;
  const int g = h / (a.heads / a.kv_heads);
  const int p = a.positions[t];
  const int* bt = a.block_tables + static_cast<long long>(a.seq_of_tok[t]) * a.max_blocks;
  const int lo = a.chunk > 0 ? p / a.chunk * a.chunk : max(0, p - a.window + 1);   // first key of the token's chunk, or of its window
  const int nk = min(a.keep_first, lo);      // kept first tokens outside the window
  const int n = nk + (p - lo + 1);
  float* qs = sm;
  float* part = sm + ((D + 3) & ~3);
  for (int d = threadIdx.x; d < D; d += blockDim.x) qs[d] = a.qn[(t * a.heads + h) * D + d] * a.scale;
  __syncthreads();
  const long long crow = static_cast<long long>(a.kv_heads) * (D + Dv);
  const T* cache = static_cast<const T*>(a.cache);
  const long long koff = static_cast<long long>(g) * D, voff = static_cast<long long>(a.kv_heads) * D + static_cast<long long>(g) * Dv;
  float m = -FLT_MAX, l = 0.f, acc[kMaxVR];
#pragma unroll
  for (int r = 0; r < kMaxVR; ++r) acc[r] = 0.f;
  for (int c0 = wrp * 32; c0 < n; c0 += nwarps * 32) {
    const int i = c0 + lane;
    long long row = -1;
    float s = -FLT_MAX;
    if (i < n) {
      const int j = i < nk ? i : lo + (i - nk);
      row = static_cast<long long>(bt[j / a.page]) * a.page + j % a.page;
      s = dot_row(qs, cache + row * crow + koff, D, vec);
      if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
    }
    float cm = s;
    for (int o = 16; o > 0; o >>= 1) cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, o));
    const float mn = fmaxf(m, cm);
    const float corr = expf(m - mn);
    const float pr = i < n ? expf(s - mn) : 0.f;
    float ps = pr;
    for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
    l = fmaf(l, corr, ps);
    m = mn;
#pragma unroll
    for (int r = 0; r < kMaxVR; ++r) acc[r] *= corr;
    const int cn = min(32, n - c0);
    for (int kk = 0; kk < cn; ++kk) {
      const float pk = __shfl_sync(0xffffffffu, pr, kk);
      const long long rk = __shfl_sync(0xffffffffu, row, kk);
      const T* vp = cache + rk * crow + voff;
#pragma unroll
      for (int r = 0; r < kMaxVR; ++r) {
        const int c = lane + 32 * r;
        if (c < Dv) acc[r] = fmaf(pk, ldf(vp + c), acc[r]);
      }
    }
  }
  // the warps' partial (m, l, acc) meet in shared memory and are merged in warp order
  float* mine = part + wrp * (Dv + 2);
  if (lane == 0) { mine[0] = m; mine[1] = l; }
#pragma unroll
  for (int r = 0; r < kMaxVR; ++r) {
    const int c = lane + 32 * r;
    if (c < Dv) mine[2 + c] = acc[r];
  }
  __syncthreads();
  // the sink adds exp(sink) to the denominator and nothing to the numerator; it is taken as it is, outside scale and cap
  const float sink = a.sink ? a.sink[h] : -FLT_MAX;
  float mm = sink;
  for (int w = 0; w < nwarps; ++w) mm = fmaxf(mm, part[w * (Dv + 2)]);
  float ll = a.sink ? expf(sink - mm) : 0.f;
  float f[kWarpsDecode];
#pragma unroll
  for (int w = 0; w < kWarpsDecode; ++w) f[w] = 0.f;
#pragma unroll
  for (int w = 0; w < kWarpsDecode; ++w) {
    if (w >= nwarps) break;
    const float pm = part[w * (Dv + 2)];
    f[w] = pm == -FLT_MAX ? 0.f : expf(pm - mm);
    ll = fmaf(part[w * (Dv + 2) + 1], f[w], ll);
  }
  const float inv = 1.0f / ll;
  const T* gate = static_cast<const T*>(a.gate);
  T* y = static_cast<T*>(a.y) + t * a.ldy + static_cast<long long>(h) * Dv;
  for (int c = threadIdx.x; c < Dv; c += blockDim.x) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < kWarpsDecode; ++w)
      if (w < nwarps) o = fmaf(part[w * (Dv + 2) + 2 + c], f[w], o);
    o *= inv;
    if (gate) o *= sigmoidf_(ldf(gate + t * a.ldg + (a.gate_per_head ? h : static_cast<long long>(h) * Dv + c)));
    stf(y + c, o * a.out_scale);
  }
}

// ---------------------------------------------------------------------------------------------- attention on the tensor cores
// bf16 cache, dim % 16 == 0, vdim % 16 == 0, both <= 128.  A CTA of four warps owns 64 query rows of one sequence: TQ = 64 / gs
// consecutive tokens times the gs query heads that share one key/value head (gs = heads / kv_heads when that divides 64,
// else 1 and every query head is its own group), so one key/value tile in shared memory serves the whole group.  Keys
// come in tiles of 64 from the pages by cp.async into one key and one value buffer (three CTAs fit an SM): the next keys
// are copied under the softmax and the second product, the next values under the next scores; first come the kept first
// tokens that lie before the tile's
// lowest window, then the window itself.  S = Q K^T and O += P V are mma.sync m16n8k16 products with fp32 accumulators;
// the mask (j <= p, p - j < window or j < keep_first, per row), the scale and the online softmax work on the score
// fragments in registers (fp32; the exponentials are the fast fp32 intrinsic, as bf16 serving allows), a row's four lanes share
// its maximum by shuffles.  P is rounded to bf16 for the second product.
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void ldsm_x4(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

constexpr int kTileRows = 64, kTileKeys = 64, kMmaThreads = 2 * kTileRows, kMmaCtasPerSm = 3;
constexpr float kMasked = -1e30f;

template <int NV>   // value n-tiles of 8 columns held per thread: vdim <= 8 * NV
__global__ void __launch_bounds__(kMmaThreads, kMmaCtasPerSm) window_attn_mma_kernel(WindowAttnArgs a, int gs, int TQ, int page_shift) {
  extern __shared__ __align__(16) unsigned char smraw[];
  __shared__ long long rowoff[kTileKeys];                // cache row (in elements) of every key of a tile, looked up once
  const int D = a.dim, Dv = a.vdim, LDK = D + 8, LDV = Dv + 8;
  bf16* Qs = reinterpret_cast<bf16*>(smraw);                 // [rows][LDK]
  bf16* Ks = Qs + kTileRows * LDK;                           // [64][LDK]
  bf16* Vs = Ks + kTileKeys * LDK;                           // [64][LDV]
  const int tid = threadIdx.x, lane = tid & 31, wrp = tid >> 5, g = lane >> 2, t4 = lane & 3;
  // which sequence and which tile of it
  int tile = blockIdx.x, s = 0, n = 0;
  for (; s < a.nseq; ++s) {
    n = a.seqs[s * 8 + 1];
    const int nt = (n + TQ - 1) / TQ;
    if (tile < nt) { tile = nt - 1 - tile; break; }   // a sequence's last tiles see the most keys: they start first
    tile -= nt;
  }
  if (s >= a.nseq) return;
  const int tok0 = a.seqs[s * 8] + tile * TQ, ntq = min(TQ, n - tile * TQ);
  const int p0 = a.seqs[s * 8 + 2] + tile * TQ, p1 = p0 + ntq - 1;
  const int hy = blockIdx.y;                                // group of query heads
  const int kvh = (hy * gs) / (a.heads / a.kv_heads);
  const int* bt = a.block_tables + static_cast<long long>(s) * a.max_blocks;
  const long long crow = static_cast<long long>(a.kv_heads) * (D + Dv);
  const bf16* cache = static_cast<const bf16*>(a.cache);
  const long long koff = static_cast<long long>(kvh) * D, voff = static_cast<long long>(a.kv_heads) * D + static_cast<long long>(kvh) * Dv;
  // queries -> bf16 rows (row r: token r / gs, head hy * gs + r % gs); a warp takes rows wrp, wrp + warps, ...
  for (int r = wrp; r < kTileRows; r += kMmaThreads / 32) {
    const int tq = r / gs, hh = r - tq * gs;
    const float* src = a.qn + (static_cast<long long>(tok0 + tq) * a.heads + hy * gs + hh) * D;
    for (int c = 2 * lane; c < D; c += 64) {
      float2 v = make_float2(0.f, 0.f);
      if (tq < ntq) v = *reinterpret_cast<const float2*>(src + c);
      *reinterpret_cast<uint32_t*>(Qs + r * LDK + c) = pack_bf16(v.x, v.y);
    }
  }
  // the first key a row at position p sees besides the kept first tokens: the start of its chunk, or of its window
  auto first_key = [&](int p) { return a.chunk > 0 ? p / a.chunk * a.chunk : max(0, p - a.window + 1); };
  const int lo0 = first_key(p0);
  const int nsink = min(a.keep_first, lo0);
  const int nst = (nsink + kTileKeys - 1) / kTileKeys;
  const int nwt = (p1 - lo0 + 1 + kTileKeys - 1) / kTileKeys;
  const int ntiles = nst + nwt;
  const int kchunks = D / 8, chunks = kchunks + Dv / 8;      // 16-byte pieces of a key row and of a key + value row
  auto tile_range = [&](int i, int* j0, int* cnt) {
    if (i < nst) { *j0 = i * kTileKeys; *cnt = min(kTileKeys, nsink - *j0); }
    else { *j0 = lo0 + (i - nst) * kTileKeys; *cnt = min(kTileKeys, p1 + 1 - *j0); }
  };
  auto lookup_rows = [&](int i) {     // threads 0..63: the cache row of tile i's keys
    if (tid < kTileKeys && i < ntiles) {
      int j0, cnt;
      tile_range(i, &j0, &cnt);
      const int j = j0 + min(tid, cnt - 1);    // rows past the range repeat its last key: finite values under a zero weight
      const long long slot = page_shift >= 0 ? (static_cast<long long>(bt[j >> page_shift]) << page_shift) + (j & ((1 << page_shift) - 1))
                                             : static_cast<long long>(bt[j / a.page]) * a.page + j % a.page;
      rowoff[tid] = slot * crow;
    }
  };
  // Keys and values of a tile are copied separately (the key buffer is free again after the scores, the value buffer after
  // the second product).  The (row, piece) a thread copies first and its step to its next piece: no division per tile.
  const int vchunks = chunks - kchunks;
  const int kr_first = tid / kchunks, kc_first = tid - kr_first * kchunks, kr_step = kMmaThreads / kchunks, kc_step = kMmaThreads - kr_step * kchunks;
  const int vr_first = tid / vchunks, vc_first = tid - vr_first * vchunks, vr_step = kMmaThreads / vchunks, vc_step = kMmaThreads - vr_step * vchunks;
  auto load_keys = [&]() {
    int r = kr_first, c = kc_first;
    while (r < kTileKeys) {
      cp_async16(smem_u32(Ks + r * LDK + c * 8), cache + rowoff[r] + koff + c * 8);
      r += kr_step; c += kc_step;
      if (c >= kchunks) { c -= kchunks; ++r; }
    }
    cp_async_commit();
  };
  auto load_values = [&]() {
    int r = vr_first, c = vc_first;
    while (r < kTileKeys) {
      cp_async16(smem_u32(Vs + r * LDV + c * 8), cache + rowoff[r] + voff + c * 8);
      r += vr_step; c += vc_step;
      if (c >= vchunks) { c -= vchunks; ++r; }
    }
    cp_async_commit();
  };
  float m[2] = {kMasked, kMasked}, l[2] = {0.f, 0.f};
  float o[NV][4];
#pragma unroll
  for (int i = 0; i < NV; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  const int nv = Dv / 8;
  // this thread's two rows
  int prow[2], plo[2];
  bool rowok[2];
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    const int r = 16 * wrp + g + 8 * hf, tq = r / gs;
    prow[hf] = p0 + tq;
    plo[hf] = first_key(prow[hf]);
    rowok[hf] = tq < ntq;
  }
  lookup_rows(0);
  __syncthreads();
  // the positions of the warp's 16 rows, for the whole-tile test
  const int warp_pmin = p0 + (16 * wrp) / gs, warp_pmax = p0 + (16 * wrp + 15) / gs;
  const bool warp_ok = (16 * wrp + 15) / gs < ntq;
  const int warp_lo = first_key(warp_pmax);   // the latest first key among the warp's rows
  // shared-memory addresses of this lane's ldmatrix rows, formed once: the loops below only add multiples of a k-step
  const uint32_t q_base = smem_u32(Qs + (16 * wrp + (lane & 7) + ((lane >> 3) & 1) * 8) * LDK + (lane >> 4) * 8);
  const uint32_t k_base = smem_u32(Ks + ((lane & 7) + (lane >> 4) * 8) * LDK + ((lane >> 3) & 1) * 8);
  const uint32_t v_base = smem_u32(Vs + ((lane & 7) + ((lane >> 3) & 1) * 8) * LDV + (lane >> 4) * 8);
  const uint32_t k_blk = 16 * LDK * sizeof(bf16), v_blk = 16 * LDV * sizeof(bf16);
  load_keys();
  load_values();
  for (int i = 0; i < ntiles; ++i) {
    cp_async_wait<1>();        // this tile's keys have landed (its values may still be on their way)
    __syncthreads();
    lookup_rows(i + 1);        // every copy of tile i has been issued: the row table is free for the next tile
    int j0, cnt;
    tile_range(i, &j0, &cnt);
    float sc[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) { sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f; }
#pragma unroll 2
    for (int ks = 0; ks < 2 * D; ks += 32) {      // byte offset of the k-step
      uint32_t af[4];
      ldsm_x4(af, q_base + ks);
#pragma unroll
      for (int nb = 0; nb < 4; ++nb) {
        uint32_t bfr[4];
        ldsm_x4(bfr, k_base + nb * k_blk + ks);
        mma_bf16(sc[2 * nb], af, bfr[0], bfr[1]);
        mma_bf16(sc[2 * nb + 1], af, bfr[2], bfr[3]);
      }
    }
    __syncthreads();           // the key buffer is free, the next tile's row table is written
    const bool more = i + 1 < ntiles;
    if (more) load_keys();     // the next keys arrive under the softmax and the second product
    // mask, scale, running maximum.  A tile that every row of the warp sees whole (all keys at or before the warp's
    // first position and inside its last row's window) needs no per-element test.
    float mx[2] = {kMasked, kMasked};
    if (a.softcap > 0.f) {
      // score <- cap * tanh(scale * score / cap), tanh(z) = 1 - 2 / (exp(2 z) + 1); the scale that follows is then 1
      const float pre = 2.0f * a.scale / a.softcap;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) sc[nt][e] = a.softcap * (1.0f - __fdividef(2.0f, __expf(sc[nt][e] * pre) + 1.0f));
    }
    const float sscale = a.softcap > 0.f ? 1.0f : a.scale;
    const bool whole = cnt == kTileKeys && warp_ok && j0 + kTileKeys - 1 <= warp_pmin && (j0 >= warp_lo || j0 + kTileKeys <= a.keep_first);
    if (whole) {
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float v = sc[nt][e] * sscale;
          sc[nt][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
    } else {
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int hf = e >> 1, col = nt * 8 + 2 * t4 + (e & 1), j = j0 + col, p = prow[hf];
          const bool vis = rowok[hf] && col < cnt && j <= p && (j >= plo[hf] || j < a.keep_first);
          const float v = vis ? sc[nt][e] * sscale : kMasked;
          sc[nt][e] = v;
          mx[hf] = fmaxf(mx[hf], v);
        }
    }
    float corr[2];
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      mx[hf] = fmaxf(mx[hf], __shfl_xor_sync(0xffffffffu, mx[hf], 1));
      mx[hf] = fmaxf(mx[hf], __shfl_xor_sync(0xffffffffu, mx[hf], 2));
      const float mn = fmaxf(m[hf], mx[hf]);
      corr[hf] = __expf(m[hf] - mn);     // 1 while the row has seen nothing (both at the sentinel)
      m[hf] = mn;
      l[hf] *= corr[hf];
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int hf = e >> 1;
        const float pv = sc[nt][e] <= kMasked ? 0.f : __expf(sc[nt][e] - m[hf]);
        sc[nt][e] = pv;
        l[hf] += pv;
      }
#pragma unroll
    for (int i2 = 0; i2 < NV; ++i2) { o[i2][0] *= corr[0]; o[i2][1] *= corr[0]; o[i2][2] *= corr[1]; o[i2][3] *= corr[1]; }
    // O += P V
    if (more) cp_async_wait<1>(); else cp_async_wait<0>();     // this tile's values
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t pf[4];
      pf[0] = pack_bf16(sc[2 * kk][0], sc[2 * kk][1]);
      pf[1] = pack_bf16(sc[2 * kk][2], sc[2 * kk][3]);
      pf[2] = pack_bf16(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
      pf[3] = pack_bf16(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
#pragma unroll
      for (int nb = 0; nb < NV / 2; ++nb) {
        if (2 * nb < nv) {
          uint32_t bfr[4];
          ldsm_x4_trans(bfr, v_base + kk * v_blk + nb * 32);
          mma_bf16(o[2 * nb], pf, bfr[0], bfr[1]);
          mma_bf16(o[2 * nb + 1], pf, bfr[2], bfr[3]);
        }
      }
    }
    __syncthreads();           // the value buffer is free
    if (more) load_values();   // the next values arrive under the next tile's scores
    else cp_async_commit();    // keeps the count of groups in flight the same on the last round
  }
  // finish: row sums over the four lanes of a row, gate, branch scale, one rounding
  const bf16* gate = static_cast<const bf16*>(a.gate);
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    float ls = l[hf];
    ls += __shfl_xor_sync(0xffffffffu, ls, 1);
    ls += __shfl_xor_sync(0xffffffffu, ls, 2);
    if (!rowok[hf]) continue;
    const int r = 16 * wrp + g + 8 * hf, tq = r / gs, hh = r - tq * gs;
    const long long t = tok0 + tq;
    const int head = hy * gs + hh;
    float inv = 1.0f / ls;
    if (a.sink) {
      // the sink's term joins the denominator only: move the reference point if the sink lies above it
      const float sk = a.sink[head], mn = fmaxf(m[hf], sk), back = __expf(m[hf] - mn);
      inv = back / (ls * back + __expf(sk - mn));
    }
    bf16* y = static_cast<bf16*>(a.y) + t * a.ldy + static_cast<long long>(head) * Dv;
#pragma unroll
    for (int i2 = 0; i2 < NV; ++i2) {
      if (i2 < nv) {
        const int c = 8 * i2 + 2 * t4;
        float v0 = o[i2][2 * hf] * inv, v1 = o[i2][2 * hf + 1] * inv;
        if (gate && a.gate_per_head) {
          const float sg = sigmoidf_(__bfloat162float(gate[t * a.ldg + head]));
          v0 *= sg; v1 *= sg;
        } else if (gate) {
          const __nv_bfloat162 gv = *reinterpret_cast<const __nv_bfloat162*>(gate + t * a.ldg + static_cast<long long>(head) * Dv + c);
          v0 *= sigmoidf_(__bfloat162float(gv.x));
          v1 *= sigmoidf_(__bfloat162float(gv.y));
        }
        *reinterpret_cast<uint32_t*>(y + c) = pack_bf16(v0 * a.out_scale, v1 * a.out_scale);
      }
    }
  }
}

}  // namespace

int rope_table_yarn(float2* table, int max_pos, int dims, double base, const RopeYarn* yarn, cudaStream_t st) {
  const int half = dims / 2;
  if (max_pos <= 0 || half <= 0) return 0;
  if (!(base > 0.0) || (yarn && !(yarn->factor > 0.0 && yarn->original > 0.0 && yarn->fast > 0.0 && yarn->slow > 0.0))) return -1;
  const double pi = 3.14159265358979323846;
  double lo = 0, hi = 0, mag = 1.0;
  if (yarn) {
    auto at = [&](double turns) { return dims * log(yarn->original / (2.0 * pi * turns)) / (2.0 * log(base)); };
    lo = std::max(floor(at(yarn->fast)), 0.0);
    hi = std::min(ceil(at(yarn->slow)), static_cast<double>(dims - 1));
    mag = 0.1 * log(yarn->factor) + 1.0;
  }
  std::vector<float2> h(static_cast<size_t>(max_pos) * half);
  for (int i = 0; i < half; ++i) {
    double f = pow(base, -2.0 * i / dims);
    if (yarn) {
      const double ramp = std::min(1.0, std::max(0.0, (i - lo) / std::max(hi - lo, 0.001)));
      f = f / yarn->factor * ramp + f * (1.0 - ramp);
    }
    for (int p = 0; p < max_pos; ++p) {
      const double ang = p * f;
      h[static_cast<size_t>(p) * half + i] = make_float2(static_cast<float>(cos(ang) * mag), static_cast<float>(sin(ang) * mag));
    }
  }
  if (cudaMemcpyAsync(table, h.data(), h.size() * sizeof(float2), cudaMemcpyHostToDevice, st) != cudaSuccess) return -2;
  return cudaStreamSynchronize(st) == cudaSuccess ? 0 : -2;
}

int qk_rope_norm_cache(const QkPrepArgs& a, cudaStream_t st) {
  if (a.T <= 0) return 0;
  if (a.heads < 1 || a.kv_heads < 1 || a.dim < 1 || a.vdim < 1 || a.rot_dims < 0 || a.rot_dims > a.dim || a.rot_dims % 2 || (a.rot_dims && !a.rope)) return -1;
  if (a.t == DT_BF16) qk_prep_kernel<bf16><<<a.T, 128, 0, st>>>(a);
  else qk_prep_kernel<float><<<a.T, 128, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int conv_qk_prep(const ConvQkPrepArgs& a, cudaStream_t st) {
  if (a.T <= 0) return 0;
  if (!a.qk || !a.qn || !a.cache || a.heads < 1 || a.kv_heads < 1 || a.dim < 1 || a.rot_dims < 0 || a.rot_dims > a.dim || a.rot_dims % 2 ||
      (a.rot_dims && !a.rope) || (a.conv_w && (a.taps < 1 || (a.taps > 1 && !a.conv_state))) || !a.seqs || !a.seq_of_tok) return -1;
  const int C = (a.heads + a.kv_heads) * a.dim;
  const size_t smem = static_cast<size_t>(C) * sizeof(float);
  static std::atomic<unsigned long long> set16{0}, set32{0};
  if (smem > 200 * 1024) return -1;
  // steps of few tokens leave most SMs idle, so a token's CTA is as wide as its row allows (a thread per channel up to the
  // CTA's limit); steps of many tokens keep more CTAs per SM with narrower ones
  const int th = a.T >= 256 ? (C >= 2048 ? 256 : 128) : std::min(1024, std::max(128, (C + 31) / 32 * 32));
  if (a.t == DT_BF16) {
    if (smem > 48 * 1024 && !ensure_dynamic_smem(conv_qk_prep_kernel<bf16>, 200 * 1024, &set16)) return -2;
    conv_qk_prep_kernel<bf16><<<a.T, th, smem, st>>>(a);
  } else {
    if (smem > 48 * 1024 && !ensure_dynamic_smem(conv_qk_prep_kernel<float>, 200 * 1024, &set32)) return -2;
    conv_qk_prep_kernel<float><<<a.T, th, smem, st>>>(a);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int window_attention(const WindowAttnArgs& a, cudaStream_t st) {
  if (a.T <= 0) return 0;
  if (a.heads < 1 || a.kv_heads < 1 || a.heads % a.kv_heads || a.dim < 1 || a.vdim < 1 || a.vdim > 32 * kMaxVR || (a.chunk <= 0 && a.window < 1) || a.keep_first < 0 ||
      a.page < 1) return -1;
  // Steps that bring portions of prompts take the tensor-core kernel when the head sizes fit its fragments; steps of
  // single tokens (and every fp32 model) take the general kernel.  B200_WATTN_MMA=0 / 1 forces the choice (A/B knob).
  const char* fe = getenv("B200_WATTN_MMA");
  const int force = fe ? atoi(fe) : -1;
  const bool fits = a.t == DT_BF16 && a.dim % 16 == 0 && a.vdim % 16 == 0 && a.dim <= 128 && a.vdim <= 128 && a.seqs && a.nseq > 0 && a.ldy % 2 == 0 &&
                    (!a.gate || a.gate_per_head || a.ldg % 2 == 0) && reinterpret_cast<uintptr_t>(a.cache) % 16 == 0;
  const bool want = force >= 0 ? force != 0 : (a.T >= 32 && a.T >= 8 * a.nseq);
  if (fits && want) {
    const int group = a.heads / a.kv_heads;
    const int gs = kTileRows % group == 0 ? group : 1;
    const int TQ = kTileRows / gs;
    int page_shift = -1;
    for (int b = 0; b < 31; ++b) if ((1 << b) == a.page) page_shift = b;
    const size_t smem = (static_cast<size_t>(kTileRows + kTileKeys) * (a.dim + 8) + static_cast<size_t>(kTileKeys) * (a.vdim + 8)) * sizeof(bf16);
    dim3 grid(static_cast<unsigned>((a.T + TQ - 1) / TQ + a.nseq), static_cast<unsigned>(a.heads / gs));
    static std::atomic<unsigned long long> set8{0}, set16{0};
    if (a.vdim <= 64) {
      if (!ensure_dynamic_smem(window_attn_mma_kernel<8>, 112 * 1024, &set8)) return -2;
      cudaFuncSetAttribute(window_attn_mma_kernel<8>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
      window_attn_mma_kernel<8><<<grid, kMmaThreads, smem, st>>>(a, gs, TQ, page_shift);
    } else {
      if (!ensure_dynamic_smem(window_attn_mma_kernel<16>, 112 * 1024, &set16)) return -2;
      cudaFuncSetAttribute(window_attn_mma_kernel<16>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
      window_attn_mma_kernel<16><<<grid, kMmaThreads, smem, st>>>(a, gs, TQ, page_shift);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
  }
  const int vl = a.t == DT_BF16 ? 8 : 4;
  const bool vec = a.dim % vl == 0 && (static_cast<long long>(a.kv_heads) * (a.dim + a.vdim)) % vl == 0 && reinterpret_cast<uintptr_t>(a.cache) % 16 == 0;
  // single-token steps of few sequences: more warps per (token, head) shorten the chain of key chunks a warp walks
  const int warps = static_cast<long long>(a.T) * a.heads <= 1024 ? kWarpsDecode : kWarps;
  const size_t smem = (static_cast<size_t>((a.dim + 3) & ~3) + warps * (a.vdim + 2)) * sizeof(float);
  if (smem > 48 * 1024) return -1;
  const unsigned grid = static_cast<unsigned>(static_cast<long long>(a.T) * a.heads);
  if (a.t == DT_BF16) window_attn_kernel<bf16><<<grid, warps * 32, smem, st>>>(a, vec);
  else window_attn_kernel<float><<<grid, warps * 32, smem, st>>>(a, vec);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // namespace b200
