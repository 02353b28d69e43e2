// Elementwise kernels of the fp32-residual model designs (mixers.h): hashed bigram embedding, Dynamic-Tanh norm fused
// with the residual update that precedes it, the (optionally clamped) gated unit, bias + activation in place, a sigmoid
// output gate and an fp32 argmax.
// Every transcendental is evaluated in fp32 with the accurate library functions (tanhf, expf), not the fast intrinsics:
// the same kernels serve the fp32 model mode.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>

#include "mixers.h"

namespace b200 {
namespace {

typedef __nv_bfloat16 bf16;
__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const bf16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(bf16* p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }

template <typename TW>
__global__ void embed_bigram_kernel(const TW* embed, const TW* bigram, const int* ids, const int* prev_ids, float* x, int W, int vocab,
                                    int buckets, long long mul_prev, long long mul_cur) {
  const int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const int prev = prev_ids[t];
  const long long row = prev < 0 ? buckets : (static_cast<long long>(prev) * mul_prev + static_cast<long long>(id) * mul_cur) % buckets;
  const TW* e = embed + static_cast<long long>(id) * W;
  const TW* g = bigram + row * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) x[static_cast<long long>(t) * W + i] = ldf(e + i) + ldf(g + i);
}

template <typename TA, typename TY>
__global__ void residual_dyt_kernel(float* x, const TA* a, const TA* f, float mult, const float* w, const float* b, const float* alpha,
                                    TY* y, const int* row_index, int W) {
  const int r = blockIdx.x;
  const long long t = row_index ? row_index[r] : r;
  const float al = y ? alpha[0] : 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float v = x[t * W + i];
    if (a || f) {
      float s = 0.f;
      if (a) s += ldf(a + t * W + i);
      if (f) s += ldf(f + t * W + i);
      v = fmaf(mult, s, v);
      x[t * W + i] = v;
    }
    if (y) stf(y + static_cast<long long>(r) * W + i, fmaf(tanhf(al * v), w[i], b[i]));
  }
}

template <typename T>
__global__ void glu_clamped_kernel(const T* gu, int ldgu, T* y, int ldy, int F, float limit, float slope, float up_offset, long long total) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / F;
  const int c = static_cast<int>(i - t * F);
  const float g = fminf(ldf(gu + t * ldgu + c), limit);
  const float u = fminf(fmaxf(ldf(gu + t * ldgu + F + c), -limit), limit);
  stf(y + t * ldy + c, g * sigmoidf_(slope * g) * (u + up_offset));
}

template <typename T>
__global__ void bias_act_kernel(T* y, int ldy, const float* bias, int act, int n, long long total) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / n;
  const int c = static_cast<int>(i - t * n);
  float v = ldf(y + t * ldy + c) + (bias ? bias[c] : 0.f);
  if (act == LIN_RELU2) { v = fmaxf(v, 0.f); v = v * v; }
  stf(y + t * ldy + c, v);
}

template <typename T>
__global__ void sigmoid_gate_kernel(T* y, int ldy, const T* g, int ldg, int n, long long total) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / n;
  const int c = static_cast<int>(i - t * n);
  stf(y + t * ldy + c, ldf(y + t * ldy + c) * sigmoidf_(ldf(g + t * ldg + c)));
}

__global__ void argmax_f32_kernel(const float* logits, int* out, int V) {
  __shared__ float bv[32];
  __shared__ int bi[32];
  const float* row = logits + static_cast<long long>(blockIdx.x) * V;
  float best = -FLT_MAX;
  int idx = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    if (v > best) { best = v; idx = i; }   // i ascending per thread: the first maximum wins
  }
  auto better = [](float v, int i, float bv_, int bi_) { return v > bv_ || (v == bv_ && i < bi_); };
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (better(ov, oi, best, idx)) { best = ov; idx = oi; }
  }
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5;
  if (lane == 0) { bv[wrp] = best; bi[wrp] = idx; }
  __syncthreads();
  if (wrp == 0) {
    const int nw = blockDim.x >> 5;
    best = lane < nw ? bv[lane] : -FLT_MAX;
    idx = lane < nw ? bi[lane] : 0x7fffffff;
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (better(ov, oi, best, idx)) { best = ov; idx = oi; }
    }
    if (lane == 0) out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;
  }
}

template <typename T>
__global__ void fill_uniform_kernel(T* p, size_t n, uint64_t seed, float scale, float offset) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  // splitmix64 of (seed, i)
  uint64_t z = seed + 0x9E3779B97F4A7C15ull * (i + 1);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  const float u = static_cast<float>(z >> 40) * (2.0f / 16777216.0f) - 1.0f;
  stf(p + i, fmaf(scale, u, offset));
}

inline int done() { return cudaGetLastError() == cudaSuccess ? 0 : -2; }
inline int threads_for(int W) { return W >= 1024 ? 256 : (W >= 256 ? 128 : 64); }

}  // namespace

int embed_bigram(const void* embed, const void* bigram, DType tw, const int* ids, const int* prev_ids, float* x, int T, int W, int vocab,
                 int buckets, long long mul_prev, long long mul_cur, cudaStream_t st) {
  if (T <= 0) return 0;
  if (buckets < 1 || W < 1) return -1;
  if (tw == DT_BF16)
    embed_bigram_kernel<bf16><<<T, threads_for(W), 0, st>>>(static_cast<const bf16*>(embed), static_cast<const bf16*>(bigram), ids, prev_ids, x, W, vocab, buckets, mul_prev, mul_cur);
  else
    embed_bigram_kernel<float><<<T, threads_for(W), 0, st>>>(static_cast<const float*>(embed), static_cast<const float*>(bigram), ids, prev_ids, x, W, vocab, buckets, mul_prev, mul_cur);
  return done();
}

int residual_dyt(float* x, const void* a, const void* f, DType ta, float mult, const float* w, const float* b, const float* alpha, void* y,
                 DType ty, const int* row_index, int rows, int W, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (y && (!w || !b || !alpha)) return -1;
  const int th = threads_for(W);
#define RD(TA, TY) residual_dyt_kernel<TA, TY><<<rows, th, 0, st>>>(x, static_cast<const TA*>(a), static_cast<const TA*>(f), mult, w, b, alpha, static_cast<TY*>(y), row_index, W)
  if (ta == DT_BF16 && ty == DT_BF16) RD(bf16, bf16);
  else if (ta == DT_BF16) RD(bf16, float);
  else if (ty == DT_BF16) RD(float, bf16);
  else RD(float, float);
#undef RD
  return done();
}

int glu_clamped(const void* gu, int ldgu, void* y, int ldy, DType t, int T, int F, float limit, float slope, cudaStream_t st, float up_offset) {
  const long long total = static_cast<long long>(T) * F;
  if (total <= 0) return 0;
  const unsigned grid = static_cast<unsigned>((total + 255) / 256);
  if (t == DT_BF16) glu_clamped_kernel<bf16><<<grid, 256, 0, st>>>(static_cast<const bf16*>(gu), ldgu, static_cast<bf16*>(y), ldy, F, limit, slope, up_offset, total);
  else glu_clamped_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(gu), ldgu, static_cast<float*>(y), ldy, F, limit, slope, up_offset, total);
  return done();
}

int bias_act(void* y, int ldy, const float* bias, int act, DType t, int T, int n, cudaStream_t st) {
  const long long total = static_cast<long long>(T) * n;
  if (total <= 0) return 0;
  const unsigned grid = static_cast<unsigned>((total + 255) / 256);
  if (t == DT_BF16) bias_act_kernel<bf16><<<grid, 256, 0, st>>>(static_cast<bf16*>(y), ldy, bias, act, n, total);
  else bias_act_kernel<float><<<grid, 256, 0, st>>>(static_cast<float*>(y), ldy, bias, act, n, total);
  return done();
}

int sigmoid_gate(void* y, int ldy, const void* g, int ldg, DType t, int T, int n, cudaStream_t st) {
  const long long total = static_cast<long long>(T) * n;
  if (total <= 0) return 0;
  const unsigned grid = static_cast<unsigned>((total + 255) / 256);
  if (t == DT_BF16) sigmoid_gate_kernel<bf16><<<grid, 256, 0, st>>>(static_cast<bf16*>(y), ldy, static_cast<const bf16*>(g), ldg, n, total);
  else sigmoid_gate_kernel<float><<<grid, 256, 0, st>>>(static_cast<float*>(y), ldy, static_cast<const float*>(g), ldg, n, total);
  return done();
}

int fill_uniform(void* p, DType t, size_t n, uint64_t seed, float scale, float offset, cudaStream_t st) {
  if (!n) return 0;
  const unsigned grid = static_cast<unsigned>((n + 255) / 256);
  if (t == DT_BF16) fill_uniform_kernel<bf16><<<grid, 256, 0, st>>>(static_cast<bf16*>(p), n, seed, scale, offset);
  else fill_uniform_kernel<float><<<grid, 256, 0, st>>>(static_cast<float*>(p), n, seed, scale, offset);
  return done();
}

int argmax_f32(const float* logits, int* out, int S, int V, cudaStream_t st) {
  if (S <= 0) return 0;
  argmax_f32_kernel<<<S, 256, 0, st>>>(logits, out, V);
  return done();
}

}  // namespace b200
