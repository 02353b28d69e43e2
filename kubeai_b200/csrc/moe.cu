// Mixture-of-experts plumbing (mixers.h): group-limited routing on fp32 scores, a counting sort of the (token, choice)
// pairs into expert-grouped 64-row tiles for the grouped launches of linear.cu, and the weighted combine.
//
// Routing of one token: s = softmax(z) over all E experts; the experts form `groups` equal groups of neighbours, a group
// is ranked by its largest s, only the `keep` best groups stay eligible; the `top` largest eligible s win, ties to the
// lower index, and s itself (not renormalised) is the weight.  Other forms score by sigmoid(z) alone, or rank by z and
// weight the winners by the softmax over the winners' z only.  A pair's result never depends on which other pairs
// share its tile, and the combine adds a token's choices in the order the router picked them.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>

#include "mixers.h"

namespace b200 {
namespace {

typedef __nv_bfloat16 bf16;

// one warp per token; scores row in global memory is the scratch (chosen entries are overwritten with -1)
__global__ void moe_route_kernel(float* scores, int* topk_ids, float* topk_w, int T, int E, int groups, int keep, int top, int score_fn, int ld,
                                 const float* bias) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  const int lane = threadIdx.x & 31;
  float* s = scores + static_cast<long long>(t) * ld;
  // scores of the other forms lie in [0, 1]; raw logits may be anything, so their "nothing yet" mark is the lowest float
  const float none = score_fn == MOE_TOP_SOFTMAX ? -FLT_MAX : -1.f;
  if (score_fn == MOE_SIGMOID) {
    for (int e = lane; e < E; e += 32) s[e] = 1.0f / (1.0f + expf(-s[e]));
  } else if (score_fn == MOE_TOP_SOFTMAX) {
    for (int e = lane; e < E; e += 32) s[e] = fmaxf(s[e], -0.5f * FLT_MAX);   // a logit stays above the mark
  } else {
    float mx = -FLT_MAX;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, s[e]);
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) { const float v = expf(s[e] - mx); s[e] = v; sum += v; }
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.0f / sum;
    for (int e = lane; e < E; e += 32) s[e] *= inv;
  }
  __syncwarp();
  // with a selection bias the experts are ranked by score + bias (a chosen entry, marked, ranks below everything) and
  // weighted by the score itself
  const float lowest = bias ? -FLT_MAX : none;
  auto rank = [&](int e) { const float v = s[e]; return bias ? (v == none ? -FLT_MAX : v + bias[e]) : v; };
  const int per = E / groups;
  // keep the best groups: bit g of `kept` (lane-uniform); groups <= 64
  unsigned long long kept = 0;
  for (int r = 0; r < keep; ++r) {
    float best = lowest;
    int bg = 0x7fffffff;
    for (int g = lane; g < groups; g += 32) {
      if (kept >> g & 1ull) continue;
      float gm = lowest;
      for (int e = g * per; e < (g + 1) * per; ++e) gm = fmaxf(gm, rank(e));
      if (gm > best) { best = gm; bg = g; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int og = __shfl_xor_sync(0xffffffffu, bg, o);
      if (ob > best || (ob == best && og < bg)) { best = ob; bg = og; }
    }
    if (bg != 0x7fffffff) kept |= 1ull << bg;
  }
  float first = 0.f, sum = 0.f;   // MOE_TOP_SOFTMAX: the largest chosen logit and the sum of exp(logit - first) over the chosen
  for (int k = 0; k < top; ++k) {
    float best = lowest;
    int be = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      if (!(kept >> (e / per) & 1ull)) continue;
      const float v = rank(e);
      if (v > best) { best = v; be = e; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ob > best || (ob == best && oe < be)) { best = ob; be = oe; }
    }
    if (be == 0x7fffffff) { be = 0; best = 0.f; }
    else if (bias) best = s[be];     // the weight is the score without the bias
    if (k == 0) first = best;
    sum += expf(best - first);
    if (lane == 0) {
      topk_ids[static_cast<long long>(t) * top + k] = be;
      topk_w[static_cast<long long>(t) * top + k] = best;
      s[be] = none;
    }
    __syncwarp();
  }
  if (score_fn == MOE_TOP_SOFTMAX) {
    const float inv = 1.0f / sum;
    for (int k = lane; k < top; k += 32) {
      float* w = topk_w + static_cast<long long>(t) * top + k;
      *w = expf(*w - first) * inv;
    }
  }
}

// single CTA: histogram, padded offsets, scatter
__global__ void __launch_bounds__(1024) moe_align_kernel(const int* topk_ids, int pairs, int top, int E, int* sorted_rows, int* tile_group,
                                                         int* pair_pos, int cap, int* expert_rows, const float* topk_w, float* sorted_w, int matrices) {
  extern __shared__ int sh[];   // count[E], start[E + 1], fill[E]
  int* count = sh;
  int* start = sh + E;
  int* fill = sh + 2 * E + 1;
  for (int e = threadIdx.x; e < E; e += blockDim.x) { count[e] = 0; fill[e] = 0; }
  for (int i = threadIdx.x; i < cap; i += blockDim.x) { sorted_rows[i] = -1; if (sorted_w) sorted_w[i] = 0.f; }
  for (int i = threadIdx.x; i < cap / 64; i += blockDim.x) tile_group[i] = -1;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) atomicAdd(&count[topk_ids[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) {
      start[e] = at;
      if (expert_rows) { expert_rows[2 * e] = at; expert_rows[2 * e + 1] = count[e]; }
      const int tiles = (count[e] + 63) / 64;
      for (int i = 0; i < tiles; ++i) tile_group[at / 64 + i] = e < matrices ? e : -1;   // an expert without matrices: its tiles are skipped
      at += tiles * 64;
    }
    start[E] = at;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = topk_ids[p];
    const int r = start[e] + atomicAdd(&fill[e], 1);
    sorted_rows[r] = p / top;
    pair_pos[p] = r;
    if (sorted_w) sorted_w[r] = topk_w[p];
  }
}

__device__ __forceinline__ float ldy(const float* p) { return *p; }
__device__ __forceinline__ float ldy(const bf16* p) { return __bfloat162float(*p); }

// ids with matrices and x (optional): a choice at or above `matrices` is an identity expert, whose output is the token's
// row of x itself; its row of y was never written and is not read.
template <typename T, typename TYIN>
__global__ void moe_combine_kernel(const TYIN* y, const int* pair_pos, const float* topk_w, T* out, int top, int W, const T* add = nullptr,
                                   const float* add_gate = nullptr, int ld_gate = 0, const int* ids = nullptr, int matrices = 0,
                                   const T* x = nullptr) {
  const long long t = blockIdx.x;
  float gate = 1.f;
  if (add && add_gate) gate = 1.0f / (1.0f + expf(-add_gate[t * ld_gate]));
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k) {
      const float yv = (ids && ids[t * top + k] >= matrices) ? ldy(x + t * W + i) : ldy(y + static_cast<long long>(pair_pos[t * top + k]) * W + i);
      acc = topk_w ? fmaf(topk_w[t * top + k], yv, acc) : acc + yv;
    }
    if (add) acc = fmaf(gate, ldy(add + t * W + i), acc);
    if (sizeof(T) == 2) reinterpret_cast<bf16*>(out)[t * W + i] = __float2bfloat16_rn(acc);
    else reinterpret_cast<float*>(out)[t * W + i] = acc;
  }
}

}  // namespace

int moe_route(float* scores, int* topk_ids, float* topk_w, int T, int E, int groups, int keep, int top, cudaStream_t st, int score_fn, int ld,
              const float* select_bias) {
  if (T <= 0) return 0;
  if (E < 1 || groups < 1 || groups > 64 || E % groups || keep < 1 || keep > groups || top < 1 || top > keep * (E / groups)) return -1;
  if (select_bias && score_fn == MOE_TOP_SOFTMAX) return -1;
  moe_route_kernel<<<(T + 3) / 4, 128, 0, st>>>(scores, topk_ids, topk_w, T, E, groups, keep, top, score_fn, ld > 0 ? ld : E, select_bias);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int moe_align(const int* topk_ids, int T, int top, int E, int* sorted_rows, int* tile_group, int* pair_pos, int cap, cudaStream_t st,
              int* expert_rows, const float* topk_w, float* sorted_w, int matrices) {
  if (T <= 0) return 0;
  if (cap % 64 || cap < T * top + E * 64 || (sorted_w && !topk_w)) return -1;
  const size_t smem = static_cast<size_t>(3 * E + 1) * sizeof(int);
  if (smem > 48 * 1024) return -1;
  moe_align_kernel<<<1, 1024, smem, st>>>(topk_ids, T * top, top, E, sorted_rows, tile_group, pair_pos, cap, expert_rows, topk_w, sorted_w, matrices > 0 ? matrices : E);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int moe_combine(const void* y, DType ty, const int* pair_pos, const float* topk_w, void* out, DType t, int T, int top, int W, cudaStream_t st) {
  if (T <= 0) return 0;
  const int th = W >= 1024 ? 256 : 128;
  if (ty == DT_BF16) {
    if (t != DT_BF16) return -1;
    moe_combine_kernel<bf16, bf16><<<T, th, 0, st>>>(static_cast<const bf16*>(y), pair_pos, topk_w, static_cast<bf16*>(out), top, W);
  } else if (t == DT_BF16) moe_combine_kernel<bf16, float><<<T, th, 0, st>>>(static_cast<const float*>(y), pair_pos, topk_w, static_cast<bf16*>(out), top, W);
  else moe_combine_kernel<float, float><<<T, th, 0, st>>>(static_cast<const float*>(y), pair_pos, topk_w, static_cast<float*>(out), top, W);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int moe_combine_add(const void* y, DType ty, const int* pair_pos, const float* topk_w, const void* add, const float* add_gate, int ld_gate,
                    void* out, DType t, int T, int top, int W, cudaStream_t st) {
  if (T <= 0) return 0;
  if (!y || !pair_pos || !out || top < 1 || (ty == DT_BF16 && t != DT_BF16)) return -1;
  const int th = W >= 1024 ? 256 : 128;
  if (ty == DT_BF16)
    moe_combine_kernel<bf16, bf16><<<T, th, 0, st>>>(static_cast<const bf16*>(y), pair_pos, topk_w, static_cast<bf16*>(out), top, W,
                                                       static_cast<const bf16*>(add), add_gate, ld_gate);
  else if (t == DT_BF16)
    moe_combine_kernel<bf16, float><<<T, th, 0, st>>>(static_cast<const float*>(y), pair_pos, topk_w, static_cast<bf16*>(out), top, W,
                                                        static_cast<const bf16*>(add), add_gate, ld_gate);
  else
    moe_combine_kernel<float, float><<<T, th, 0, st>>>(static_cast<const float*>(y), pair_pos, topk_w, static_cast<float*>(out), top, W,
                                                         static_cast<const float*>(add), add_gate, ld_gate);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int moe_combine_identity(const void* y, DType ty, const int* pair_pos, const float* topk_w, const int* topk_ids, int matrices, const void* x,
                         void* out, DType t, int T, int top, int W, cudaStream_t st) {
  if (T <= 0) return 0;
  if (!y || !pair_pos || !topk_ids || !x || !out || top < 1 || matrices < 0 || (ty == DT_BF16 && t != DT_BF16)) return -1;
  const int th = W >= 1024 ? 256 : 128;
  if (ty == DT_BF16)
    moe_combine_kernel<bf16, bf16><<<T, th, 0, st>>>(static_cast<const bf16*>(y), pair_pos, topk_w, static_cast<bf16*>(out), top, W, nullptr, nullptr, 0,
                                                       topk_ids, matrices, static_cast<const bf16*>(x));
  else if (t == DT_BF16)
    moe_combine_kernel<bf16, float><<<T, th, 0, st>>>(static_cast<const float*>(y), pair_pos, topk_w, static_cast<bf16*>(out), top, W, nullptr, nullptr, 0,
                                                        topk_ids, matrices, static_cast<const bf16*>(x));
  else
    moe_combine_kernel<float, float><<<T, th, 0, st>>>(static_cast<const float*>(y), pair_pos, topk_w, static_cast<float*>(out), top, W, nullptr, nullptr, 0,
                                                         topk_ids, matrices, static_cast<const float*>(x));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

namespace {
// rows of x in expert-sorted order (16-byte pieces; W % 8 == 0): a negative source row becomes zeros
__global__ void moe_gather_kernel(const uint4* x, const int* sorted_rows, uint4* out, int pieces, long long total, const float* row_scale) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long r = i / pieces;
  const int c = static_cast<int>(i - r * pieces);
  const int src = sorted_rows[r];
  uint4 v = src < 0 ? make_uint4(0, 0, 0, 0) : x[static_cast<long long>(src) * pieces + c];
  if (row_scale && src >= 0) {
    const float s = row_scale[r];
    uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const __nv_bfloat162 o = __floats2bfloat162_rn(__uint_as_float(u[k] << 16) * s, __uint_as_float(u[k] & 0xffff0000u) * s);
      u[k] = *reinterpret_cast<const uint32_t*>(&o);
    }
    v = make_uint4(u[0], u[1], u[2], u[3]);
  }
  out[i] = v;
}
__global__ void relu2_kernel(__nv_bfloat162* p, long long n2) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n2) return;
  float2 v = __bfloat1622float2(p[i]);
  v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f);
  p[i] = __floats2bfloat162_rn(v.x * v.x, v.y * v.y);
}
}  // namespace

int moe_gather_bf16(const void* x, const int* sorted_rows, void* out, int rows, int W, cudaStream_t st, const float* row_scale) {
  if (rows <= 0) return 0;
  if (W % 8) return -1;
  const long long total = static_cast<long long>(rows) * (W / 8);
  moe_gather_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, st>>>(static_cast<const uint4*>(x), sorted_rows, static_cast<uint4*>(out), W / 8, total, row_scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int relu2_bf16(void* p, long long n, cudaStream_t st) {
  if (n <= 0) return 0;
  if (n % 2) return -1;
  relu2_kernel<<<static_cast<unsigned>((n / 2 + 255) / 256), 256, 0, st>>>(static_cast<__nv_bfloat162*>(p), n / 2);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // namespace b200
