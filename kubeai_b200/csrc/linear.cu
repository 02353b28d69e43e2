// Shape-agnostic linear layer: Y = act(X W^T + bias) for any T, N, K, in bf16 or fp32 storage with fp32 accumulation.
// Three uses share one kernel family (mixers.h LinearArgs): a plain projection, one projection per head inside wider
// rows (batch index = head), and expert-grouped rows (64-row tiles that each name their weight matrix).  It is the
// projection path of every shape the tcgen05 GEMMs (gemm2_tcgen05.cu: bf16, K % 8 == 0, bf16 output) do not take:
// fp32 models, fp32 outputs (router logits, decay pre-activations, latent queries), odd sizes, gathers.
//
// Kernels: a 64 x 64 x 32 shared-memory tile kernel (fp32 weights: FMA, k ascending; bf16 weights: mma.sync tensor-core
// products; either way one output element is accumulated in an order that does not depend on what else is in the batch), and a one-warp-per-output-row kernel for steps of at most 8 rows (decode), which
// streams each weight row once with 16-byte loads.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "mixers.h"

namespace b200 {
namespace {

typedef __nv_bfloat16 bf16;
constexpr int BM = 64, BN = 64, BK = 32;

__device__ __forceinline__ float ld1(const float* p) { return *p; }
__device__ __forceinline__ float ld1(const bf16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void st1(float* p, float v) { *p = v; }
__device__ __forceinline__ void st1(bf16* p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ void ld8(const float* p, float* o) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
__device__ __forceinline__ void ld8(const bf16* p, float* o) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    o[2 * i] = __uint_as_float(u[i] << 16);
    o[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ float apply_act(float v, int act) {
  if (act == LIN_RELU2) { v = fmaxf(v, 0.f); v = v * v; }
  return v;
}

template <typename TX, typename TW, typename TY>
__global__ void __launch_bounds__(256) linear_tile_kernel(LinearArgs a) {
  __shared__ float Xs[BM][BK + 1];
  __shared__ float Ws[BN][BK + 1];
  const int tid = threadIdx.x, lane = tid & 31, wrp = tid >> 5;
  const int row0 = blockIdx.y * BM, col0 = blockIdx.x * BN;
  const long long b = blockIdx.z;
  const TX* X = static_cast<const TX*>(a.X) + b * a.xbs;
  const TW* W = static_cast<const TW*>(a.W) + b * a.wbs;
  TY* Y = static_cast<TY*>(a.Y) + b * a.ybs;
  if (a.tile_group) {
    const int g = a.tile_group[blockIdx.y];
    if (g < 0) return;
    W += static_cast<long long>(g) * a.wbs;
  }
  // the 8 rows of X and of W this thread stages per k-tile (row = warp + 8 i, column = lane)
  long long xoff[8], woff[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = wrp + 8 * i;
    int t = row0 + r;
    if (t >= a.T) t = -1;
    else if (a.x_rows) t = a.x_rows[t];
    xoff[i] = t < 0 ? -1 : static_cast<long long>(t) * a.ldx;
    const int n = col0 + r;
    woff[i] = n < a.N ? static_cast<long long>(n) * a.ldw : -1;
  }
  const int ty = tid >> 4, tx = tid & 15;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < a.K; k0 += BK) {
    const int k = k0 + lane;
    const bool kin = k < a.K;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int r = wrp + 8 * i;
      Xs[r][lane] = (kin && xoff[i] >= 0) ? ld1(X + xoff[i] + k) : 0.f;
      Ws[r][lane] = (kin && woff[i] >= 0) ? ld1(W + woff[i] + k) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float xv[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { xv[i] = Xs[ty * 4 + i][kk]; wv[i] = Ws[tx * 4 + i][kk]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = row0 + ty * 4 + i;
    if (t >= a.T) continue;
    if (a.x_rows && a.x_rows[t] < 0) continue;
    const float rs = a.row_scale ? a.row_scale[t] : 1.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = col0 + tx * 4 + j;
      if (n < a.N) st1(Y + static_cast<long long>(t) * a.ldy + n, apply_act((a.row_scale ? acc[i][j] * rs : acc[i][j]) + (a.bias ? a.bias[n] : 0.f), a.act));
    }
  }
}

// bf16 weights: the same 64 x 64 x 32 tile with the products on the tensor cores (mma.sync m16n8k16, fp32 accumulators).
// X is staged as bf16 (an fp32 X is rounded here); 8 warps = 4 row blocks x 2 column halves, a warp owns 16 rows x 32 columns.
__device__ __forceinline__ void mma_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ bf16 to_bf16(float v) { return __float2bfloat16_rn(v); }
__device__ __forceinline__ bf16 to_bf16(bf16 v) { return v; }

// VEC: every row start and K are multiples of 8 elements and 16-byte aligned, so a thread stages one 8-element piece of X
// and one of W per k-tile with 16-byte loads (thread -> row tid / 4, columns 8 (tid % 4) ...).
template <typename TX, typename TY, bool VEC>
__global__ void __launch_bounds__(256) linear_tile_mma_kernel(LinearArgs a) {
  constexpr int LD = BK + 8;   // 80-byte rows: the 8 rows of a fragment fall into distinct banks
  __shared__ __align__(16) bf16 Xs[BM][LD];
  __shared__ __align__(16) bf16 Ws[BN][LD];
  const int tid = threadIdx.x, lane = tid & 31, wrp = tid >> 5;
  const int row0 = blockIdx.y * BM, col0 = blockIdx.x * BN;
  const long long b = blockIdx.z;
  const TX* X = static_cast<const TX*>(a.X) + b * a.xbs;
  const bf16* W = static_cast<const bf16*>(a.W) + b * a.wbs;
  TY* Y = static_cast<TY*>(a.Y) + b * a.ybs;
  if (a.tile_group) {
    const int g = a.tile_group[blockIdx.y];
    if (g < 0) return;
    W += static_cast<long long>(g) * a.wbs;
  }
  long long xoff[8], woff[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = wrp + 8 * i;
    int t = row0 + r;
    if (t >= a.T) t = -1;
    else if (a.x_rows) t = a.x_rows[t];
    xoff[i] = t < 0 ? -1 : static_cast<long long>(t) * a.ldx;
    const int n = col0 + r;
    woff[i] = n < a.N ? static_cast<long long>(n) * a.ldw : -1;
  }
  const int wm = wrp & 3, wn = wrp >> 2, g = lane >> 2, t4 = lane & 3;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const bf16 zero = __float2bfloat16_rn(0.f);
  // vector staging: this thread's row and column piece
  const int vr = tid >> 2, vc = (tid & 3) * 8;
  long long vx = -1, vw = -1;
  if (VEC) {
    int t = row0 + vr;
    if (t >= a.T) t = -1;
    else if (a.x_rows) t = a.x_rows[t];
    vx = t < 0 ? -1 : static_cast<long long>(t) * a.ldx;
    vw = col0 + vr < a.N ? static_cast<long long>(col0 + vr) * a.ldw : -1;
  }
  for (int k0 = 0; k0 < a.K; k0 += BK) {
    if (VEC) {
      const bool kin = k0 + vc < a.K;   // K is a multiple of 8: a piece is inside or outside as a whole
      uint4 xv = make_uint4(0, 0, 0, 0), wv = make_uint4(0, 0, 0, 0);
      if (kin && vw >= 0) wv = *reinterpret_cast<const uint4*>(W + vw + k0 + vc);
      if (kin && vx >= 0) {
        if constexpr (sizeof(TX) == 2) {
          xv = *reinterpret_cast<const uint4*>(X + vx + k0 + vc);
        } else {
          const float4 f0 = *reinterpret_cast<const float4*>(X + vx + k0 + vc), f1 = *reinterpret_cast<const float4*>(X + vx + k0 + vc + 4);
          __nv_bfloat162 p0 = __floats2bfloat162_rn(f0.x, f0.y), p1 = __floats2bfloat162_rn(f0.z, f0.w);
          __nv_bfloat162 p2 = __floats2bfloat162_rn(f1.x, f1.y), p3 = __floats2bfloat162_rn(f1.z, f1.w);
          xv = make_uint4(*reinterpret_cast<uint32_t*>(&p0), *reinterpret_cast<uint32_t*>(&p1), *reinterpret_cast<uint32_t*>(&p2), *reinterpret_cast<uint32_t*>(&p3));
        }
      }
      *reinterpret_cast<uint4*>(&Xs[vr][vc]) = xv;
      *reinterpret_cast<uint4*>(&Ws[vr][vc]) = wv;
    } else {
      const int k = k0 + lane;
      const bool kin = k < a.K;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int r = wrp + 8 * i;
        Xs[r][lane] = (kin && xoff[i] >= 0) ? to_bf16(X[xoff[i] + k]) : zero;
        Ws[r][lane] = (kin && woff[i] >= 0) ? W[woff[i] + k] : zero;
      }
    }
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < BK; ks += 16) {
      uint32_t af[4];
      af[0] = *reinterpret_cast<const uint32_t*>(&Xs[16 * wm + g][ks + 2 * t4]);
      af[1] = *reinterpret_cast<const uint32_t*>(&Xs[16 * wm + g + 8][ks + 2 * t4]);
      af[2] = *reinterpret_cast<const uint32_t*>(&Xs[16 * wm + g][ks + 2 * t4 + 8]);
      af[3] = *reinterpret_cast<const uint32_t*>(&Xs[16 * wm + g + 8][ks + 2 * t4 + 8]);
#pragma unroll
      for (int nb = 0; nb < 4; ++nb) {
        const int n = 32 * wn + 8 * nb + g;
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(&Ws[n][ks + 2 * t4]);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(&Ws[n][ks + 2 * t4 + 8]);
        mma_16816(acc[nb], af, b0, b1);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int t = row0 + 16 * wm + g + 8 * half;
    if (t >= a.T) continue;
    if (a.x_rows && a.x_rows[t] < 0) continue;
    const float rs = a.row_scale ? a.row_scale[t] : 1.f;
#pragma unroll
    for (int nb = 0; nb < 4; ++nb)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int n = col0 + 32 * wn + 8 * nb + 2 * t4 + j;
        if (n < a.N) st1(Y + static_cast<long long>(t) * a.ldy + n, apply_act((a.row_scale ? acc[nb][2 * half + j] * rs : acc[nb][2 * half + j]) + (a.bias ? a.bias[n] : 0.f), a.act));
      }
  }
}

// T <= 8 rows: one warp per output column n streams W[n, :] once and keeps the T accumulators in registers.
template <typename TX, typename TW, typename TY, int VEC>
__global__ void __launch_bounds__(256) linear_rows_kernel(LinearArgs a) {
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5;
  const int n = blockIdx.x * 8 + wrp;
  if (n >= a.N) return;
  const long long b = blockIdx.z;
  const TX* X = static_cast<const TX*>(a.X) + b * a.xbs;
  const TW* w = static_cast<const TW*>(a.W) + b * a.wbs + static_cast<long long>(n) * a.ldw;
  TY* Y = static_cast<TY*>(a.Y) + b * a.ybs;
  float acc[8];
#pragma unroll
  for (int t = 0; t < 8; ++t) acc[t] = 0.f;
  for (int k = lane * VEC; k < a.K; k += 32 * VEC) {
    float wv[VEC];
    if constexpr (VEC == 8) ld8(w + k, wv); else wv[0] = ld1(w + k);
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      if (t < a.T) {
        float xv[VEC];
        const TX* xp = X + static_cast<long long>(t) * a.ldx + k;
        if constexpr (VEC == 8) ld8(xp, xv); else xv[0] = ld1(xp);
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[t] = fmaf(xv[v], wv[v], acc[t]);
      }
    }
  }
#pragma unroll
  for (int t = 0; t < 8; ++t) {
    if (t < a.T) {
      float v = acc[t];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) st1(Y + static_cast<long long>(t) * a.ldy + n, apply_act((a.row_scale ? v * a.row_scale[t] : v) + (a.bias ? a.bias[n] : 0.f), a.act));
    }
  }
}

// A few rows that each name their own source row, destination row and weight matrix (the expert choices of a decode step):
// one warp per (row, output column) streams that matrix's row once, so the step reads every chosen expert's weights at
// streaming rate instead of walking 64-row tiles that are almost empty.
template <typename TX, typename TW, typename TY, int VEC>
__global__ void __launch_bounds__(256) linear_picked_rows_kernel(LinearArgs a, PickedRows p) {
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5;
  const int n = blockIdx.x * 8 + wrp, r = blockIdx.y;
  if (n >= a.N) return;
  if (p.group_limit > 0 && (p.groups[r] < 0 || p.groups[r] >= p.group_limit)) return;   // a choice without a weight matrix
  const long long src = p.src_rows ? p.src_rows[r] : r / p.src_div;
  const long long dst = p.dst_rows[r];
  const TX* x = static_cast<const TX*>(a.X) + src * a.ldx;
  const TW* w = static_cast<const TW*>(a.W) + static_cast<long long>(p.groups[r]) * a.wbs + static_cast<long long>(n) * a.ldw;
  float acc = 0.f;
  for (int k = lane * VEC; k < a.K; k += 32 * VEC) {
    float wv[VEC], xv[VEC];
    if constexpr (VEC == 8) { ld8(w + k, wv); ld8(x + k, xv); } else { wv[0] = ld1(w + k); xv[0] = ld1(x + k); }
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc = fmaf(xv[v], wv[v], acc);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) st1(static_cast<TY*>(a.Y) + dst * a.ldy + n, apply_act((a.row_scale ? acc * a.row_scale[r] : acc) + (a.bias ? a.bias[n] : 0.f), a.act));
}

template <typename TX, typename TW, typename TY>
int launch_picked(const LinearArgs& a, const PickedRows& p, cudaStream_t st) {
  const bool vec = a.K % 8 == 0 && a.ldx % 8 == 0 && a.ldw % 8 == 0 && a.wbs % 8 == 0 && reinterpret_cast<uintptr_t>(a.X) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(a.W) % 16 == 0;
  dim3 grid((a.N + 7) / 8, p.rows);
  if (vec) linear_picked_rows_kernel<TX, TW, TY, 8><<<grid, 256, 0, st>>>(a, p);
  else linear_picked_rows_kernel<TX, TW, TY, 1><<<grid, 256, 0, st>>>(a, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

template <typename TX, typename TW, typename TY>
int launch_linear(const LinearArgs& a, cudaStream_t st) {
  const bool few = a.T <= 8 && !a.x_rows && !a.tile_group;
  if (few) {
    const size_t ex = sizeof(TX), ew = sizeof(TW);
    const bool vec = a.K % 8 == 0 && a.ldx % 8 == 0 && a.ldw % 8 == 0 && a.xbs % 8 == 0 && a.wbs % 8 == 0 &&
                     reinterpret_cast<uintptr_t>(a.X) % (8 * ex > 16 ? 16 : 8 * ex) == 0 && reinterpret_cast<uintptr_t>(a.W) % (8 * ew > 16 ? 16 : 8 * ew) == 0;
    dim3 grid((a.N + 7) / 8, 1, a.batch);
    if (vec) linear_rows_kernel<TX, TW, TY, 8><<<grid, 256, 0, st>>>(a);
    else linear_rows_kernel<TX, TW, TY, 1><<<grid, 256, 0, st>>>(a);
  } else {
    dim3 grid((a.N + BN - 1) / BN, (a.T + BM - 1) / BM, a.batch);
    if constexpr (sizeof(TW) == 2) {
      const bool vec = a.K % 8 == 0 && a.ldx % 8 == 0 && a.ldw % 8 == 0 && a.xbs % 8 == 0 && a.wbs % 8 == 0 &&
                       reinterpret_cast<uintptr_t>(a.X) % 16 == 0 && reinterpret_cast<uintptr_t>(a.W) % 16 == 0;
      if (vec) linear_tile_mma_kernel<TX, TY, true><<<grid, 256, 0, st>>>(a);
      else linear_tile_mma_kernel<TX, TY, false><<<grid, 256, 0, st>>>(a);
    } else {
      linear_tile_kernel<TX, TW, TY><<<grid, 256, 0, st>>>(a);
    }
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // namespace

int linear(const LinearArgs& a, cudaStream_t st) {
  if (a.T <= 0 || a.N <= 0) return 0;
  if (!a.X || !a.W || !a.Y || a.K <= 0 || a.batch < 1) return -1;
  if (a.tile_group && a.T % BM) return -1;
  const int key = (a.tx == DT_F32 ? 4 : 0) | (a.tw == DT_F32 ? 2 : 0) | (a.ty == DT_F32 ? 1 : 0);
  switch (key) {
    case 0: return launch_linear<bf16, bf16, bf16>(a, st);
    case 1: return launch_linear<bf16, bf16, float>(a, st);
    case 2: return launch_linear<bf16, float, bf16>(a, st);
    case 3: return launch_linear<bf16, float, float>(a, st);
    case 4: return launch_linear<float, bf16, bf16>(a, st);
    case 5: return launch_linear<float, bf16, float>(a, st);
    case 6: return launch_linear<float, float, bf16>(a, st);
    default: return launch_linear<float, float, float>(a, st);
  }
}


int linear_picked_rows(const LinearArgs& a, const PickedRows& p, cudaStream_t st) {
  if (p.rows <= 0 || a.N <= 0) return 0;
  if (!a.X || !a.W || !a.Y || a.K <= 0 || !p.dst_rows || !p.groups || (!p.src_rows && p.src_div < 1) || a.tw != a.tx) return -1;
  if (a.tx == DT_BF16) return a.ty == DT_BF16 ? launch_picked<bf16, bf16, bf16>(a, p, st) : launch_picked<bf16, bf16, float>(a, p, st);
  return a.ty == DT_BF16 ? launch_picked<float, float, bf16>(a, p, st) : launch_picked<float, float, float>(a, p, st);
}

}  // namespace b200
