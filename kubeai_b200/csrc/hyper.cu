// Hyper-connections on fp32 residual streams, fused with the RMS norm that feeds the next sublayer (mixers.h HyperArgs),
// and the scaled embedding that fills the streams.
//
// A model with n streams keeps x_1 .. x_n instead of one residual.  A sublayer reads u = sum_s in[s] x_s, and its output
// y goes back as x_j <- sum_s mix[s, j] x_s + out[j] y, every new stream computed from the old ones.  Between two
// sublayers the write-back of the first and the read of the second touch the same rows, so one kernel does both: a CTA
// owns one token row, updates the n streams in place, keeps u in shared memory, reduces mean(u^2) in a fixed order and
// writes the normed row in the storage type of the projections.  With one stream and no mixing weights the same kernel
// is the ordinary pre-norm residual step x <- x + y; h = rmsnorm(x).  Everything is fp32 up to the single rounding of h.
//
// A gated write-back multiplies y by sigmoid(gate + bias), the gate being a projection of the sublayer's own input.
// `embed_learned_pos` fills the streams with the token's embedding row plus a learned position row; `branch_norm_sum` is
// the meeting point of two mixers that ran side by side, each RMS-normed over the width with its own weight.
//
// Beside it, for designs with one residual and a norm on BOTH sides of every sublayer (mixers.h SandwichArgs): the
// sublayer's output is RMS-normed before it is added, x <- x + norm_post(y + bias), and the next sublayer reads
// norm_pre(x); one kernel per boundary, a CTA per token row, two fixed-order reductions.  And the sinusoidal position
// embedding that fills such a residual.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <math.h>

#include <vector>

#include "mixers.h"

namespace b200 {
namespace {

typedef __nv_bfloat16 bf16;
constexpr int kMaxStreams = 8;
__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const bf16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

template <typename TW>
__global__ void embed_scaled_kernel(const TW* embed, const int* ids, float* x, int W, int vocab, float scale, int streams, long long stride) {
  const long long t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const TW* e = embed + static_cast<long long>(id) * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = ldf(e + i) * scale;
    for (int s = 0; s < streams; ++s) x[s * stride + t * W + i] = v;
  }
}

// the gate of a gated write-back: sigmoid(pre-activation + bias) of column i of token t, in fp32
__device__ __forceinline__ float gate_at(const HyperArgs& a, long long t, int i) {
  const long long at = t * a.ldg + i;
  const float z = (a.tg == DT_BF16 ? __bfloat162float(static_cast<const bf16*>(a.gate)[at]) : static_cast<const float*>(a.gate)[at]) +
                  (a.gate_bias ? a.gate_bias[i] : 0.f);
  return 1.0f / (1.0f + expf(-z));
}

template <typename TY, typename TH>
__global__ void hyper_step_kernel(HyperArgs a) {
  extern __shared__ float us[];   // [W] the sublayer input before the norm
  __shared__ float red[32];
  __shared__ float coef[kMaxStreams * kMaxStreams + 2 * kMaxStreams];
  const int r = blockIdx.x, n = a.streams;
  const long long t = a.row_index ? a.row_index[r] : r;
  float* mixs = coef;
  float* outs = coef + kMaxStreams * kMaxStreams;
  float* ins = outs + kMaxStreams;
  if (threadIdx.x < n * n) mixs[threadIdx.x] = a.mix ? a.mix[threadIdx.x] : (threadIdx.x / n == threadIdx.x % n ? 1.f : 0.f);
  if (threadIdx.x < n) {
    outs[threadIdx.x] = a.out ? a.out[threadIdx.x] : 1.f;
    ins[threadIdx.x] = a.in ? a.in[threadIdx.x] : 1.f;
  }
  __syncthreads();
  const TY* y = static_cast<const TY*>(a.y);
  const bool plain = !a.mix;   // identity mixing: x_j + out[j] y exactly, without the multiplications by 0 and 1
  float ss = 0.f;
  for (int i = threadIdx.x; i < a.W; i += blockDim.x) {
    float xs[kMaxStreams];
#pragma unroll
    for (int s = 0; s < kMaxStreams; ++s)
      if (s < n) xs[s] = a.x[s * a.stream_stride + t * a.W + i];
    if (y) {
      float yv = ldf(y + t * a.W + i);
      if (a.gate) yv *= gate_at(a, t, i);
      float nx[kMaxStreams];
#pragma unroll
      for (int j = 0; j < kMaxStreams; ++j) {
        if (j < n) {
          float acc;
          if (plain) acc = xs[j];
          else {
            acc = 0.f;
#pragma unroll
            for (int s = 0; s < kMaxStreams; ++s)
              if (s < n) acc = fmaf(mixs[s * n + j], xs[s], acc);
          }
          nx[j] = fmaf(outs[j], yv, acc);
        }
      }
#pragma unroll
      for (int j = 0; j < kMaxStreams; ++j)
        if (j < n) { xs[j] = nx[j]; a.x[j * a.stream_stride + t * a.W + i] = nx[j]; }
    }
    if (a.h) {
      float u = 0.f;
      if (a.in) {
#pragma unroll
        for (int s = 0; s < kMaxStreams; ++s)
          if (s < n) u = fmaf(ins[s], xs[s], u);
      } else {
#pragma unroll
        for (int s = 0; s < kMaxStreams; ++s)
          if (s < n) u += xs[s];
      }
      us[i] = u;
      ss = fmaf(u, u, ss);
    }
  }
  if (!a.h) return;
  TH* h = static_cast<TH*>(a.h) + static_cast<long long>(r) * a.W;
  if (!a.norm_w) {
    for (int i = threadIdx.x; i < a.W; i += blockDim.x) stf(h + i, us[i]);   // each thread reads back what it wrote
    return;
  }
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5;
  if (lane == 0) red[wrp] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < (blockDim.x >> 5); ++w) tot += red[w];   // warps in a fixed order, the same in every thread
  const float inv = 1.0f / sqrtf(tot / static_cast<float>(a.W) + a.eps);
  for (int i = threadIdx.x; i < a.W; i += blockDim.x) stf(h + i, us[i] * inv * a.norm_w[i]);
}

// The same boundary for W % 4 == 0: a thread owns four neighbouring columns per round (16-byte loads and stores of the
// streams, 8-byte ones of bf16 rows).
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const bf16* p) {
  const uint2 v = *reinterpret_cast<const uint2*>(p);
  return make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u), __uint_as_float(v.y << 16), __uint_as_float(v.y & 0xffff0000u));
}
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(bf16* p, float4 v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}

template <typename TY, typename TH>
__global__ void __launch_bounds__(256) hyper_step_vec_kernel(HyperArgs a) {
  extern __shared__ __align__(16) float us[];
  __shared__ float red[32];
  __shared__ float coef[kMaxStreams * kMaxStreams + 2 * kMaxStreams];
  const int r = blockIdx.x, n = a.streams;
  const long long t = a.row_index ? a.row_index[r] : r;
  float* mixs = coef;
  float* outs = coef + kMaxStreams * kMaxStreams;
  float* ins = outs + kMaxStreams;
  if (threadIdx.x < n * n) mixs[threadIdx.x] = a.mix ? a.mix[threadIdx.x] : (threadIdx.x / n == threadIdx.x % n ? 1.f : 0.f);
  if (threadIdx.x < n) {
    outs[threadIdx.x] = a.out ? a.out[threadIdx.x] : 1.f;
    ins[threadIdx.x] = a.in ? a.in[threadIdx.x] : 1.f;
  }
  __syncthreads();
  const TY* y = static_cast<const TY*>(a.y);
  const bool plain = !a.mix;
  float ss = 0.f;
  for (int i = threadIdx.x * 4; i < a.W; i += blockDim.x * 4) {
    float xs[kMaxStreams][4];
#pragma unroll
    for (int s = 0; s < kMaxStreams; ++s)
      if (s < n) { const float4 v = ld4(a.x + s * a.stream_stride + t * a.W + i); xs[s][0] = v.x; xs[s][1] = v.y; xs[s][2] = v.z; xs[s][3] = v.w; }
    if (y) {
      const float4 y4 = ld4(y + t * a.W + i);
      float yv[4] = {y4.x, y4.y, y4.z, y4.w};
      if (a.gate) {
#pragma unroll
        for (int c = 0; c < 4; ++c) yv[c] *= gate_at(a, t, i + c);
      }
      float nx[kMaxStreams][4];
#pragma unroll
      for (int j = 0; j < kMaxStreams; ++j) {
        if (j < n) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            float acc;
            if (plain) acc = xs[j][c];
            else {
              acc = 0.f;
#pragma unroll
              for (int s = 0; s < kMaxStreams; ++s)
                if (s < n) acc = fmaf(mixs[s * n + j], xs[s][c], acc);
            }
            nx[j][c] = fmaf(outs[j], yv[c], acc);
          }
        }
      }
#pragma unroll
      for (int j = 0; j < kMaxStreams; ++j)
        if (j < n) {
#pragma unroll
          for (int c = 0; c < 4; ++c) xs[j][c] = nx[j][c];
          st4(a.x + j * a.stream_stride + t * a.W + i, make_float4(nx[j][0], nx[j][1], nx[j][2], nx[j][3]));
        }
    }
    if (a.h) {
      float u[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float v = 0.f;
        if (a.in) {
#pragma unroll
          for (int s = 0; s < kMaxStreams; ++s)
            if (s < n) v = fmaf(ins[s], xs[s][c], v);
        } else {
#pragma unroll
          for (int s = 0; s < kMaxStreams; ++s)
            if (s < n) v += xs[s][c];
        }
        u[c] = v;
        ss = fmaf(v, v, ss);
      }
      st4(us + i, make_float4(u[0], u[1], u[2], u[3]));
    }
  }
  if (!a.h) return;
  TH* h = static_cast<TH*>(a.h) + static_cast<long long>(r) * a.W;
  if (!a.norm_w) {
    for (int i = threadIdx.x * 4; i < a.W; i += blockDim.x * 4) st4(h + i, ld4(us + i));
    return;
  }
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5;
  if (lane == 0) red[wrp] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < (blockDim.x >> 5); ++w) tot += red[w];
  const float inv = 1.0f / sqrtf(tot / static_cast<float>(a.W) + a.eps);
  for (int i = threadIdx.x * 4; i < a.W; i += blockDim.x * 4) {
    const float4 u = ld4(us + i), w = ld4(a.norm_w + i);
    st4(h + i, make_float4(u.x * inv * w.x, u.y * inv * w.y, u.z * inv * w.z, u.w * inv * w.w));
  }
}

template <typename TW>
__global__ void embed_learned_pos_kernel(const TW* embed, const TW* pos_table, const int* ids, const int* pos, float* x, int W, int vocab, int max_pos,
                                         int streams, long long stride) {
  const long long t = blockIdx.x;
  int id = ids[t], p = pos[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  p = p < 0 ? 0 : (p >= max_pos ? max_pos - 1 : p);
  const TW* e = embed + static_cast<long long>(id) * W;
  const TW* pr = pos_table + static_cast<long long>(p) * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = ldf(e + i) + ldf(pr + i);
    for (int s = 0; s < streams; ++s) x[s * stride + t * W + i] = v;
  }
}

// one CTA per token: both branches' sums of squares in one pass (warps added in a fixed order), then the weighted sum
template <typename T, typename TY>
__global__ void __launch_bounds__(256) branch_norm_sum_kernel(BranchNormArgs a) {
  __shared__ float red[2][8];
  const long long t = blockIdx.x;
  const T* pa = static_cast<const T*>(a.a) + t * a.W;
  const T* pb = static_cast<const T*>(a.b) + t * a.W;
  float sa = 0.f, sb = 0.f;
  for (int i = threadIdx.x; i < a.W; i += blockDim.x) {
    const float va = ldf(pa + i), vb = ldf(pb + i);
    sa = fmaf(va, va, sa);
    sb = fmaf(vb, vb, sb);
  }
  for (int o = 16; o > 0; o >>= 1) { sa += __shfl_xor_sync(0xffffffffu, sa, o); sb += __shfl_xor_sync(0xffffffffu, sb, o); }
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5;
  if (lane == 0) { red[0][wrp] = sa; red[1][wrp] = sb; }
  __syncthreads();
  float ta = 0.f, tb = 0.f;
  for (int w = 0; w < (blockDim.x >> 5); ++w) { ta += red[0][w]; tb += red[1][w]; }
  const float ia = 1.0f / sqrtf(ta / static_cast<float>(a.W) + a.eps), ib = 1.0f / sqrtf(tb / static_cast<float>(a.W) + a.eps);
  TY* y = static_cast<TY*>(a.y) + t * a.W;
  for (int i = threadIdx.x; i < a.W; i += blockDim.x) stf(y + i, a.scale * (ldf(pa + i) * ia * a.wa[i] + ldf(pb + i) * ib * a.wb[i]));
}

inline int threads_for(int W) { return W >= 2048 ? 256 : (W >= 256 ? 128 : 64); }

// x[t] = embed[id] + sinusoid(pos).  The angle p * f is formed from the two-float frequency: a = fl(p * f_hi), the
// rounding error of that product (one fma) plus p * f_lo is a correction e of a few ulps of a, and sin(a + e), cos(a + e)
// follow from the accurate sinf / cosf of a by one step of the addition formulas.
template <typename TW>
__global__ void embed_sinusoid_kernel(const TW* embed, const int* ids, const int* pos, const float2* freq, float* x, int W, int vocab) {
  const long long t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const float p = static_cast<float>(pos[t]);
  const TW* e = embed + static_cast<long long>(id) * W;
  float* xr = x + t * W;
  for (int i = threadIdx.x; 2 * i < W; i += blockDim.x) {
    const float2 f = freq[i];
    const float a = p * f.x;
    const float err = fmaf(p, f.x, -a) + p * f.y;
    float sn, cs;
    sincosf(a, &sn, &cs);
    xr[2 * i] = ldf(e + 2 * i) + fmaf(err, cs, sn);
    if (2 * i + 1 < W) xr[2 * i + 1] = ldf(e + 2 * i + 1) + fmaf(-err, sn, cs);
  }
}

// sum over the CTA of v, the same in every thread: lanes by shuffles, warps in a fixed order
__device__ __forceinline__ float cta_sum(float v, float* red) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5;
  __syncthreads();   // red may still be read from the previous sum
  if (lane == 0) red[wrp] = v;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < (blockDim.x >> 5); ++w) tot += red[w];
  return tot;
}

// VEC: four neighbouring columns per thread and round (W % 4 == 0, every row start 16-byte aligned)
template <typename TY, typename TH, bool VEC>
__global__ void __launch_bounds__(256) sandwich_step_kernel(SandwichArgs a) {
  extern __shared__ __align__(16) float row[];   // [W]: the sublayer output with its bias, then the new residual row
  __shared__ float red[8];
  const int r = blockIdx.x;
  const long long t = a.row_index ? a.row_index[r] : r;
  float* x = a.x + t * a.W;
  const TY* y = static_cast<const TY*>(a.y);
  constexpr int C = VEC ? 4 : 1;
  const int first = threadIdx.x * C, step = blockDim.x * C;
  float inv_y = 1.f;
  if (y) {
    float ss = 0.f;
    for (int i = first; i < a.W; i += step) {
      float u[4];
      if (VEC) { const float4 v = ld4(y + t * a.W + i); u[0] = v.x; u[1] = v.y; u[2] = v.z; u[3] = v.w; }
      else u[0] = ldf(y + t * a.W + i);
#pragma unroll
      for (int c = 0; c < C; ++c) {
        if (a.y_bias) u[c] += a.y_bias[i + c];
        ss = fmaf(u[c], u[c], ss);
        row[i + c] = u[c];
      }
    }
    if (a.post_w) inv_y = 1.0f / sqrtf(cta_sum(ss, red) / static_cast<float>(a.W) + a.eps);
  }
  float ss = 0.f;
  for (int i = first; i < a.W; i += step) {
    float xv[4];
    if (VEC) { const float4 v = ld4(x + i); xv[0] = v.x; xv[1] = v.y; xv[2] = v.z; xv[3] = v.w; }
    else xv[0] = x[i];
    if (y) {
#pragma unroll
      for (int c = 0; c < C; ++c) xv[c] += a.post_w ? row[i + c] * inv_y * a.post_w[i + c] : row[i + c];   // each thread reads back what it wrote
      if (VEC) st4(x + i, make_float4(xv[0], xv[1], xv[2], xv[3]));
      else x[i] = xv[0];
    }
#pragma unroll
    for (int c = 0; c < C; ++c) { ss = fmaf(xv[c], xv[c], ss); row[i + c] = xv[c]; }
  }
  if (!a.h) return;
  TH* h = static_cast<TH*>(a.h) + static_cast<long long>(r) * a.W;
  const float inv = a.pre_w ? 1.0f / sqrtf(cta_sum(ss, red) / static_cast<float>(a.W) + a.eps) : 1.f;
  for (int i = first; i < a.W; i += step) {
    if (VEC) {
      const float4 u = ld4(row + i);
      float4 w = make_float4(1.f, 1.f, 1.f, 1.f);
      if (a.pre_w) w = ld4(a.pre_w + i);
      st4(h + i, a.pre_w ? make_float4(u.x * inv * w.x, u.y * inv * w.y, u.z * inv * w.z, u.w * inv * w.w) : u);
    } else {
      stf(h + i, a.pre_w ? row[i] * inv * a.pre_w[i] : row[i]);
    }
  }
}

}  // namespace

int sinusoid_freq_table(float2* freq, int W, double base, cudaStream_t st) {
  const int pairs = (W + 1) / 2;
  if (pairs <= 0) return 0;
  if (!(base > 0.0)) return -1;
  std::vector<float2> h(pairs);
  for (int i = 0; i < pairs; ++i) {
    const double f = pow(base, -2.0 * i / W);
    const float hi = static_cast<float>(f);
    h[i] = make_float2(hi, static_cast<float>(f - static_cast<double>(hi)));
  }
  if (cudaMemcpyAsync(freq, h.data(), h.size() * sizeof(float2), cudaMemcpyHostToDevice, st) != cudaSuccess) return -2;
  return cudaStreamSynchronize(st) == cudaSuccess ? 0 : -2;
}

int embed_sinusoid(const void* embed, DType tw, const int* ids, const int* pos, const float2* freq, float* x, int T, int W, int vocab,
                   cudaStream_t st) {
  if (T <= 0) return 0;
  if (W < 1 || !freq || !pos) return -1;
  if (tw == DT_BF16) embed_sinusoid_kernel<bf16><<<T, threads_for(W), 0, st>>>(static_cast<const bf16*>(embed), ids, pos, freq, x, W, vocab);
  else embed_sinusoid_kernel<float><<<T, threads_for(W), 0, st>>>(static_cast<const float*>(embed), ids, pos, freq, x, W, vocab);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int sandwich_step(const SandwichArgs& a, cudaStream_t st) {
  if (a.rows <= 0) return 0;
  if (!a.x || a.W < 1) return -1;
  if (a.y && a.row_index) return -1;   // an update of chosen rows only would leave the residual inconsistent
  if (!a.y && !a.h) return 0;
  const size_t smem = static_cast<size_t>(a.W) * sizeof(float);
  if (smem > 48 * 1024) return -1;
  auto al16 = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  const bool vec = a.W % 4 == 0 && al16(a.x) && al16(a.y) && al16(a.h) && al16(a.y_bias) && al16(a.post_w) && al16(a.pre_w);
  const int th = vec ? (a.W >= 1024 ? 256 : (a.W >= 512 ? 128 : 64)) : threads_for(a.W);
#define SW(TY, TH) do { if (vec) sandwich_step_kernel<TY, TH, true><<<a.rows, th, smem, st>>>(a); else sandwich_step_kernel<TY, TH, false><<<a.rows, th, smem, st>>>(a); } while (0)
  const bool y16 = a.y && a.ty == DT_BF16, h16 = a.h && a.th == DT_BF16;
  if (y16 && h16) SW(bf16, bf16);
  else if (y16) SW(bf16, float);
  else if (h16) SW(float, bf16);
  else SW(float, float);
#undef SW
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int embed_scaled(const void* embed, DType tw, const int* ids, float* x, int T, int W, int vocab, float scale, int streams,
                 long long stream_stride, cudaStream_t st) {
  if (T <= 0) return 0;
  if (W < 1 || streams < 1) return -1;
  if (tw == DT_BF16) embed_scaled_kernel<bf16><<<T, threads_for(W), 0, st>>>(static_cast<const bf16*>(embed), ids, x, W, vocab, scale, streams, stream_stride);
  else embed_scaled_kernel<float><<<T, threads_for(W), 0, st>>>(static_cast<const float*>(embed), ids, x, W, vocab, scale, streams, stream_stride);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int embed_learned_pos(const void* embed, const void* pos_table, DType tw, const int* ids, const int* pos, float* x, int T, int W, int vocab,
                      int max_pos, int streams, long long stream_stride, cudaStream_t st) {
  if (T <= 0) return 0;
  if (!embed || !pos_table || W < 1 || streams < 1 || max_pos < 1) return -1;
  if (tw == DT_BF16)
    embed_learned_pos_kernel<bf16><<<T, threads_for(W), 0, st>>>(static_cast<const bf16*>(embed), static_cast<const bf16*>(pos_table), ids, pos, x, W, vocab,
                                                                 max_pos, streams, stream_stride);
  else
    embed_learned_pos_kernel<float><<<T, threads_for(W), 0, st>>>(static_cast<const float*>(embed), static_cast<const float*>(pos_table), ids, pos, x, W, vocab,
                                                                  max_pos, streams, stream_stride);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int branch_norm_sum(const BranchNormArgs& a, cudaStream_t st) {
  if (a.T <= 0) return 0;
  if (!a.a || !a.b || !a.wa || !a.wb || !a.y || a.W < 1) return -1;
  const int th = threads_for(a.W);
#define BN(T_, TY_) branch_norm_sum_kernel<T_, TY_><<<a.T, th, 0, st>>>(a)
  if (a.t == DT_BF16) { if (a.ty == DT_BF16) BN(bf16, bf16); else BN(bf16, float); }
  else { if (a.ty == DT_BF16) BN(float, bf16); else BN(float, float); }
#undef BN
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int hyper_step(const HyperArgs& a, cudaStream_t st) {
  if (a.rows <= 0) return 0;
  if (!a.x || a.streams < 1 || a.streams > kMaxStreams || a.W < 1) return -1;
  if (a.y && a.row_index) return -1;   // an update of chosen rows only would leave the streams inconsistent
  if (a.gate && (!a.y || a.ldg < a.W)) return -1;
  const size_t smem = a.h ? static_cast<size_t>(a.W) * sizeof(float) : 0;
  if (smem > 48 * 1024) return -1;
  // four columns per thread where every row start is 16-byte aligned
  const bool vec = a.W % 4 == 0 && a.stream_stride % 4 == 0 && reinterpret_cast<uintptr_t>(a.x) % 16 == 0 && reinterpret_cast<uintptr_t>(a.y) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(a.h) % 16 == 0 && reinterpret_cast<uintptr_t>(a.norm_w) % 16 == 0;
  const int th = vec ? (a.W >= 1024 ? 256 : (a.W >= 512 ? 128 : 64)) : threads_for(a.W);
#define HS(TY, TH) do { if (vec) hyper_step_vec_kernel<TY, TH><<<a.rows, th, smem, st>>>(a); else hyper_step_kernel<TY, TH><<<a.rows, th, smem, st>>>(a); } while (0)
  const bool y16 = a.y && a.ty == DT_BF16, h16 = a.h && a.th == DT_BF16;
  if (y16 && h16) HS(bf16, bf16);
  else if (y16) HS(bf16, float);
  else if (h16) HS(float, bf16);
  else HS(float, float);
#undef HS
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // namespace b200
