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
// and registers only, and the round's outputs are finished and written by all threads.  The chain is sequential in the
// token and does the same operations however the sequence was cut into steps.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>

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
constexpr int kPer = 8;        // state entries per lane
constexpr int kRound = 16;     // tokens staged per round

template <typename T>
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
    Ar[r] = in ? a.A[static_cast<long long>(c) * a.state + nn] : 0.f;
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
        S[r] = fmaf(expf(d * Ar[r]), S[r], dx * Bt[r]);
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
  int L = 1;
  while (L * kPer < a.state) L <<= 1;
  if (L > 32) return -1;   // state <= 256
  const int chans = kScanThreads / L;
  int G = kRound;
  auto smem_for = [&](int g) { return static_cast<size_t>(g) * (2 * L * kPer + 5 * chans) * sizeof(float); };
  while (G > 1 && smem_for(G) > 44 * 1024) G >>= 1;
  dim3 grid((a.inner + chans - 1) / chans, a.nseq);
  if (a.t == DT_BF16) selective_scan_kernel<bf16><<<grid, kScanThreads, smem_for(G), st>>>(a, L, G);
  else selective_scan_kernel<float><<<grid, kScanThreads, smem_for(G), st>>>(a, L, G);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // namespace b200
