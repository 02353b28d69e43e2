// Short causal convolution over time with carried inputs, and the selective scan of Mamba (mixers.h ShortConvArgs,
// SelectiveScanArgs).
//
// Convolution: y[t, c] = act(bias[c] + sum_j w[c, j] u[t - taps + 1 + j, c]) inside one sequence.  A step brings a
// portion of a sequence; the taps - 1 inputs in front of the portion are what the last step left in the sequence's state
// slot (oldest first), zeros before the sequence's start.  One thread per (token, channel) reads its taps from the
// step's own rows or from the slot; the carry kernel then moves the last taps - 1 inputs of every sequence into the slot
// (a thread per (sequence, channel) reads ahead of what it writes, so a portion shorter than taps - 1 shifts the old
// entries correctly).  Everything is fp32 up to the one rounding of y.
//
// Selective scan: per channel c the state S[c, :] over `state` indices follows S <- exp(d A[c, :]) S + d x B_t with the
// step size d = softplus(dt) of the token and channel; the output is S . C_t + D x, gated by silu(z).  A channel belongs
// to L neighbouring lanes (L a power of two, at most 32) that hold kPer state entries each in registers; a CTA walks one
// sequence's tokens in rounds: all threads stage the round's B and C rows, step sizes, d x, x and z in shared memory
// (coalesced over channels, softplus with log1pf / expf once per token and channel), the chain then touches shared memory
// and registers only (the decay exp(d A) is formed as 2^(d A log2 e) with A log2 e held in registers), and the round's outputs are finished and written by all threads.  The chain is sequential in the
// token and does the same operations however the sequence was cut into steps.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
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
__device__ __forceinline__ float softplusf_(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

template <typename TU, typename TY>
__global__ void short_conv_kernel(ShortConvArgs a) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(a.T) * a.C) return;
  const long long t = idx / a.C;
  const int c = static_cast<int>(idx - t * a.C);
  const int* sq = a.seqs + a.seq_of_tok[t] * 8;
  const int i = static_cast<int>(t) - sq[0];        // the token's index within its portion
  const bool carried = sq[2] > 0;
  const float* st = a.state + static_cast<long long>(sq[3]) * (a.taps - 1) * a.C;
  const TU* u = static_cast<const TU*>(a.u);
  float acc = a.bias ? a.bias[c] : 0.f;
  for (int j = 0; j < a.taps; ++j) {
    const int d = a.taps - 1 - j;                    // how many tokens back
    float v = 0.f;
    if (i - d >= 0) v = ldf(u + (t - d) * a.ldu + c);
    else if (carried) v = st[static_cast<long long>(a.taps - 1 + i - d) * a.C + c];
    acc = fmaf(a.w[static_cast<long long>(c) * a.taps + j], v, acc);
  }
  if (a.act == CONV_SILU) acc = siluf_(acc);
  stf(static_cast<TY*>(a.y) + t * a.ldy + c, acc);
}

// The same for rows whose starts are 16-byte aligned and up to four taps.
template <int VEC> struct VecOf;
template <> struct VecOf<8> { typedef bf16 type; };
template <> struct VecOf<4> { typedef float type; };
__device__ __forceinline__ void ldv(const bf16* p, float* v) {
  const uint4 r = *reinterpret_cast<const uint4*>(p);
  const uint32_t u[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(u[i] << 16); v[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u); }
}
__device__ __forceinline__ void ldv(const float* p, float* v) {
  const float4 r = *reinterpret_cast<const float4*>(p);
  v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
}
__device__ __forceinline__ void stv(bf16* p, const float* v) {
  uint32_t u[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) { const __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]); u[i] = *reinterpret_cast<const uint32_t*>(&b); }
  *reinterpret_cast<uint4*>(p) = make_uint4(u[0], u[1], u[2], u[3]);
}
__device__ __forceinline__ void stv(float* p, const float* v) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }

// A thread owns VEC neighbouring channels and walks TB consecutive token rows with the last TAPS - 1 inputs in registers:
// every input row is loaded once, the weights of the thread's channels once per walk.  Where the walk enters another
// sequence (or at its start) the window is filled again, from the rows before, the sequence's carried inputs or zeros.
template <int VEC, int TAPS>
__global__ void __launch_bounds__(128) short_conv_vec_kernel(ShortConvArgs a, int TB) {
  typedef typename VecOf<VEC>::type T;
  const int groups = a.C / VEC;
  const int gi = blockIdx.x * blockDim.x + threadIdx.x;
  if (gi >= groups) return;
  const int c = gi * VEC;
  const long long t0 = static_cast<long long>(blockIdx.y) * TB, t1 = min(static_cast<long long>(a.T), t0 + TB);
  const T* u = static_cast<const T*>(a.u);
  float w[TAPS][VEC], hist[TAPS > 1 ? TAPS - 1 : 1][VEC], bias[VEC], rows[4][VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    bias[e] = a.bias ? a.bias[c + e] : 0.f;
#pragma unroll
    for (int j = 0; j < TAPS; ++j) w[j][e] = a.w[static_cast<long long>(c + e) * TAPS + j];
  }
  int cur = -1;
  for (long long t = t0; t < t1; ++t) {
    const int s = a.seq_of_tok[t];
    if (s != cur) {
      // hist[k] = the input TAPS - 1 - k tokens before t
      cur = s;
      const int* sq = a.seqs + s * 8;
      const int i = static_cast<int>(t) - sq[0];
      const bool carried = sq[2] > 0;
      const float* st = a.state + static_cast<long long>(sq[3]) * (TAPS - 1) * a.C;
#pragma unroll
      for (int k = 0; k < TAPS - 1; ++k) {
        const int d = TAPS - 1 - k;
        if (i - d >= 0) ldv(u + (t - d) * a.ldu + c, hist[k]);
        else {
#pragma unroll
          for (int e = 0; e < VEC; ++e) hist[k][e] = carried ? st[static_cast<long long>(TAPS - 1 + i - d) * a.C + c + e] : 0.f;
        }
      }
    }
    // the loads of up to four rows are issued together, ahead of the arithmetic of the first
    const int q = static_cast<int>(t - t0) & 3;
    if (q == 0) {
#pragma unroll
      for (int r = 0; r < 4; ++r)
        if (t + r < t1) ldv(u + (t + r) * a.ldu + c, rows[r]);
    }
    float v[VEC], acc[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) v[e] = q == 0 ? rows[0][e] : (q == 1 ? rows[1][e] : (q == 2 ? rows[2][e] : rows[3][e]));
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      float r = bias[e];
#pragma unroll
      for (int k = 0; k < TAPS - 1; ++k) r = fmaf(w[k][e], hist[k][e], r);     // oldest tap first, the token's own last
      r = fmaf(w[TAPS - 1][e], v[e], r);
      acc[e] = a.act == CONV_SILU ? siluf_(r) : r;
    }
#pragma unroll
    for (int k = 0; k + 1 < TAPS - 1; ++k)
#pragma unroll
      for (int e = 0; e < VEC; ++e) hist[k][e] = hist[k + 1][e];
    if (TAPS > 1) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) hist[TAPS - 2][e] = v[e];
    }
    stv(static_cast<T*>(a.y) + t * a.ldy + c, acc);
  }
}

template <typename TU>
__global__ void short_conv_carry_kernel(ShortConvArgs a) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x, s = blockIdx.y;
  if (c >= a.C) return;
  const int* sq = a.seqs + s * 8;
  const int row0 = sq[0], n = sq[1];
  const bool carried = sq[2] > 0;
  float* st = a.state + static_cast<long long>(sq[3]) * (a.taps - 1) * a.C;
  const TU* u = static_cast<const TU*>(a.u);
  // entry k holds the input at portion index n - (taps - 1) + k; a negative index is the old entry k + n (read before any
  // entry at or above it is written, since k ascends)
  for (int k = 0; k < a.taps - 1; ++k) {
    const int i = n - (a.taps - 1) + k;
    float v = 0.f;
    if (i >= 0) v = ldf(u + static_cast<long long>(row0 + i) * a.ldu + c);
    else if (carried) v = st[static_cast<long long>(k + n) * a.C + c];
    st[static_cast<long long>(k) * a.C + c] = v;
  }
}

constexpr int kScanThreads = 128;
constexpr int kRound = 16;     // tokens staged per round

// kPer = state entries per lane: 8 where the step has threads enough to fill the GPU that way, 4 (twice the lanes per
// channel, half the chain per lane) where it has not
template <typename T, int kPer>
__global__ void __launch_bounds__(kScanThreads) selective_scan_kernel(SelectiveScanArgs a, int L, int G) {
  extern __shared__ float sm[];
  const int chans = kScanThreads / L, NP = L * kPer;      // channels per CTA, padded state size
  const int seq = blockIdx.y;
  const int tok0 = a.seqs[seq * 8], n = a.seqs[seq * 8 + 1], pos0 = a.seqs[seq * 8 + 2], slot = a.seqs[seq * 8 + 3];
  const int cl = threadIdx.x / L, part = threadIdx.x % L;
  const int c0 = blockIdx.x * chans, c = c0 + cl;
  const bool live = c < a.inner;
  float* Bs = sm;                    // [G][NP]
  float* Cs = Bs + G * NP;           // [G][NP]
  float* ds = Cs + G * NP;           // [G][chans] step sizes
  float* dxs = ds + G * chans;       // [G][chans] step size times x
  float* xs = dxs + G * chans;       // [G][chans]
  float* zs = xs + G * chans;        // [G][chans]
  float* ys = zs + G * chans;        // [G][chans]
  float S[kPer], Ar[kPer];
  float* Sg = a.states + (static_cast<long long>(slot) * a.inner + (live ? c : 0)) * a.state;
#pragma unroll
  for (int r = 0; r < kPer; ++r) {
    const int nn = part * kPer + r;
    const bool in = live && nn < a.state;
    Ar[r] = in ? a.A[static_cast<long long>(c) * a.state + nn] * 1.44269504088896340736f : 0.f;   // A log2(e): exp(d A) = 2^(d A log2 e)
    S[r] = (in && pos0 > 0) ? Sg[nn] : 0.f;
  }
  const T* x = static_cast<const T*>(a.x);
  const T* z = static_cast<const T*>(a.z);
  for (int g0 = 0; g0 < n; g0 += G) {
    const int gn = min(G, n - g0);
    __syncthreads();
    for (int e = threadIdx.x; e < gn * NP; e += kScanThreads) {
      const int tt = e / NP, nn = e - tt * NP;
      const float* row = a.bc + static_cast<long long>(tok0 + g0 + tt) * a.ldbc;
      Bs[e] = nn < a.state ? row[a.b_off + nn] : 0.f;
      Cs[e] = nn < a.state ? row[a.c_off + nn] : 0.f;
    }
    for (int e = threadIdx.x; e < gn * chans; e += kScanThreads) {
      const int tt = e / chans, cc = c0 + (e - tt * chans);
      const long long row = tok0 + g0 + tt;
      float d = 0.f, xv = 0.f, zv = 0.f;
      if (cc < a.inner) {
        d = softplusf_(a.dt[row * a.lddt + cc]);
        xv = ldf(x + row * a.ldx + cc);
        zv = ldf(z + row * a.ldz + cc);
      }
      ds[e] = d; dxs[e] = d * xv; xs[e] = xv; zs[e] = zv;
    }
    __syncthreads();
    for (int tt = 0; tt < gn; ++tt) {
      const float d = ds[tt * chans + cl], dx = dxs[tt * chans + cl];
      const float* Bt = Bs + tt * NP + part * kPer;
      const float* Ct = Cs + tt * NP + part * kPer;
      float acc = 0.f;
#pragma unroll
      for (int r = 0; r < kPer; ++r) {
        S[r] = fmaf(exp2f(d * Ar[r]), S[r], dx * Bt[r]);
        acc = fmaf(S[r], Ct[r], acc);
      }
      for (int o = L >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (part == 0) ys[tt * chans + cl] = acc;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < gn * chans; e += kScanThreads) {
      const int tt = e / chans, cc = c0 + (e - tt * chans);
      if (cc < a.inner) {
        const float v = fmaf(a.D[cc], xs[e], ys[e]);
        stf(static_cast<T*>(a.y) + static_cast<long long>(tok0 + g0 + tt) * a.ldy + cc, v * siluf_(zs[e]));
      }
    }
  }
  if (live) {
#pragma unroll
    for (int r = 0; r < kPer; ++r) {
      const int nn = part * kPer + r;
      if (nn < a.state) Sg[nn] = S[r];
    }
  }
}

}  // namespace

int short_conv(const ShortConvArgs& a, cudaStream_t st) {
  if (a.T <= 0) return 0;
  if (!a.u || !a.w || !a.y || a.C < 1 || a.taps < 1 || (a.taps > 1 && !a.state) || !a.seqs || !a.seq_of_tok) return -1;
  const long long total = static_cast<long long>(a.T) * a.C;
  const int vec = a.t == DT_BF16 ? 8 : 4;
  if (a.t == a.ty && a.taps >= 1 && a.taps <= 4 && a.C % vec == 0 && a.ldu % vec == 0 && a.ldy % vec == 0 && reinterpret_cast<uintptr_t>(a.u) % 16 == 0 &&
      reinterpret_cast<uintptr_t>(a.y) % 16 == 0) {
    // rows per walk: long enough to amortise the window's fill, short enough to leave every SM several CTAs
    const int groups = a.C / vec;
    int TB = 16;
    while (TB > 1 && static_cast<long long>((a.T + TB - 1) / TB) * ((groups + 127) / 128) < 4 * 148) TB >>= 1;
    dim3 vgrid((groups + 127) / 128, (a.T + TB - 1) / TB);
#define SC(V_, K_) short_conv_vec_kernel<V_, K_><<<vgrid, 128, 0, st>>>(a, TB)
    if (a.t == DT_BF16) { switch (a.taps) { case 1: SC(8, 1); break; case 2: SC(8, 2); break; case 3: SC(8, 3); break; default: SC(8, 4); } }
    else { switch (a.taps) { case 1: SC(4, 1); break; case 2: SC(4, 2); break; case 3: SC(4, 3); break; default: SC(4, 4); } }
#undef SC
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
  }
  const unsigned grid = static_cast<unsigned>((total + 255) / 256);
  if (a.t == DT_BF16) {
    if (a.ty == DT_BF16) short_conv_kernel<bf16, bf16><<<grid, 256, 0, st>>>(a);
    else short_conv_kernel<bf16, float><<<grid, 256, 0, st>>>(a);
  } else {
    if (a.ty == DT_BF16) short_conv_kernel<float, bf16><<<grid, 256, 0, st>>>(a);
    else short_conv_kernel<float, float><<<grid, 256, 0, st>>>(a);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int short_conv_carry(const ShortConvArgs& a, cudaStream_t st) {
  if (a.nseq <= 0 || a.taps <= 1) return 0;
  if (!a.u || !a.state || a.C < 1 || !a.seqs) return -1;
  dim3 grid((a.C + 127) / 128, a.nseq);
  if (a.t == DT_BF16) short_conv_carry_kernel<bf16><<<grid, 128, 0, st>>>(a);
  else short_conv_carry_kernel<float><<<grid, 128, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int selective_scan(const SelectiveScanArgs& a, cudaStream_t st) {
  if (a.nseq <= 0) return 0;
  if (!a.x || !a.z || !a.dt || !a.bc || !a.A || !a.D || !a.states || !a.y || a.inner < 1 || a.state < 1) return -1;
  int sms = 148;
  { int dev = 0; if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
  auto lanes = [&](int per) { int l = 1; while (l * per < a.state) l <<= 1; return l; };
  int per = 8;
  if (lanes(8) > 32 || (lanes(4) <= 32 && static_cast<long long>(a.nseq) * a.inner * lanes(8) < static_cast<long long>(sms) * 1536)) per = 4;
  if (const char* e = getenv("B200_SSM_PER")) per = atoi(e) == 4 ? 4 : 8;   // A/B knob
  const int L = lanes(per);
  if (L > 32) return -1;   // state <= 256
  const int chans = kScanThreads / L;
  int G = kRound;
  auto smem_for = [&](int g) { return static_cast<size_t>(g) * (2 * L * per + 5 * chans) * sizeof(float); };
  while (G > 1 && smem_for(G) > 44 * 1024) G >>= 1;
  dim3 grid((a.inner + chans - 1) / chans, a.nseq);
#define SS(T_, P_) selective_scan_kernel<T_, P_><<<grid, kScanThreads, smem_for(G), st>>>(a, L, G)
  if (a.t == DT_BF16) { if (per == 4) SS(bf16, 4); else SS(bf16, 8); }
  else { if (per == 4) SS(float, 4); else SS(float, 8); }
#undef SS
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // namespace b200
