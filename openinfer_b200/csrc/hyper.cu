// Layers over several residual streams (hyper-connections). The streams of a row are X [S, W] in float32. A sublayer
// reads u = sum_s a[s] x_s through its norm, and its result y comes back as x'_r = sum_s M[s, r] x_s + b[r] y, all r
// from the old streams. One kernel ends a sublayer and opens the next: it writes the new streams and, from them, the
// next sublayer's normed input in the model's type, as the residual add and the following norm are one kernel in the
// single-stream layers. With S = 1 and no coefficients (a = b = 1, M = 1) this is the plain pre-norm residual on a
// float32 stream.
#include "common.cuh"

namespace {

constexpr int kStreamLimit = 16;   // the kernels are built for up to 4, 8 and 16 streams

// X [rows, S, W]. Part 1 (y != null): the streams of the row are mixed and y is added (y2 != null: y = c1 y + c2 y2).
// Part 2 (out != null): out[row] = u * rsqrt(mean(u^2) + eps) * (w_offset + w), u = sum_s a[s] x_s (a null: the plain sum).
// row_idx (part 2 alone): output row r reads the streams of row row_idx[r].
// kVec: columns a thread handles side by side (4: 16-byte accesses, for widths that are a multiple of four).
template <typename TO, int kVec, int kMaxStreams>
__global__ void hyper_step_kernel(float* __restrict__ X, int S, int W, const float* __restrict__ y, const float* __restrict__ y2,
                                  float c1, float c2, const void* __restrict__ mix, const void* __restrict__ b_out,
                                  const void* __restrict__ a_in, int p_dtype, const void* __restrict__ norm_w, int nw_dtype,
                                  float eps, float w_offset, TO* __restrict__ out, const int* __restrict__ row_idx) {
  pdl_start();
  __shared__ float sM[kMaxStreams * kMaxStreams], sB[kMaxStreams], sA[kMaxStreams], red[32];
  const int row_out = blockIdx.x;
  const int row = row_idx ? row_idx[row_out] : row_out;
  if (threadIdx.x < S * S) sM[threadIdx.x] = mix ? load_as_f32(mix, p_dtype, threadIdx.x) : (threadIdx.x / S == threadIdx.x % S ? 1.f : 0.f);
  if (threadIdx.x < S) {
    sB[threadIdx.x] = b_out ? load_as_f32(b_out, p_dtype, threadIdx.x) : 1.f;
    sA[threadIdx.x] = a_in ? load_as_f32(a_in, p_dtype, threadIdx.x) : 1.f;
  }
  __syncthreads();
  float* xr = X + (size_t)row * S * W;
  auto load = [&](const float* p, float (&v)[kVec]) {
    if (kVec == 4) {
      const float4 t = *reinterpret_cast<const float4*>(p);
      v[0] = t.x, v[1] = t.y, v[2] = t.z, v[kVec - 1] = t.w;
    } else {
      v[0] = *p;
    }
  };
  auto store = [&](float* p, const float (&v)[kVec]) {
    if (kVec == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[kVec - 1]);
    else *p = v[0];
  };
  float ss = 0.f;
  for (int c = threadIdx.x * kVec; c < W; c += blockDim.x * kVec) {
    float x[kMaxStreams][kVec];
#pragma unroll
    for (int s = 0; s < kMaxStreams; ++s) {
      if (s < S) load(xr + (size_t)s * W + c, x[s]);
      else
#pragma unroll
        for (int e = 0; e < kVec; ++e) x[s][e] = 0.f;
    }
    if (y) {
      float yv[kVec];
      load(y + (size_t)row * W + c, yv);
      if (y2) {
        float y2v[kVec];
        load(y2 + (size_t)row * W + c, y2v);
#pragma unroll
        for (int e = 0; e < kVec; ++e) yv[e] = c1 * yv[e] + c2 * y2v[e];
      }
      float nx[kMaxStreams][kVec];
#pragma unroll
      for (int r = 0; r < kMaxStreams; ++r) {
#pragma unroll
        for (int e = 0; e < kVec; ++e) nx[r][e] = 0.f;
        if (r < S) {
#pragma unroll
          for (int s = 0; s < kMaxStreams; ++s)
            if (s < S)
#pragma unroll
              for (int e = 0; e < kVec; ++e) nx[r][e] += sM[s * S + r] * x[s][e];
#pragma unroll
          for (int e = 0; e < kVec; ++e) nx[r][e] += sB[r] * yv[e];
          store(xr + (size_t)r * W + c, nx[r]);
        }
      }
#pragma unroll
      for (int s = 0; s < kMaxStreams; ++s)
#pragma unroll
        for (int e = 0; e < kVec; ++e) x[s][e] = nx[s][e];
    }
    if (out) {
#pragma unroll
      for (int e = 0; e < kVec; ++e) {
        float u = 0.f;
#pragma unroll
        for (int s = 0; s < kMaxStreams; ++s)
          if (s < S) u += sA[s] * x[s][e];
        ss += u * u;
      }
    }
  }
  if (!out) return;
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / (float)W + eps);
  for (int c = threadIdx.x * kVec; c < W; c += blockDim.x * kVec) {   // the thread reads back what it wrote itself
    float u[kVec];
#pragma unroll
    for (int e = 0; e < kVec; ++e) u[e] = 0.f;
#pragma unroll
    for (int s = 0; s < kMaxStreams; ++s)
      if (s < S) {
        float xv[kVec];
        load(xr + (size_t)s * W + c, xv);
#pragma unroll
        for (int e = 0; e < kVec; ++e) u[e] += sA[s] * xv[e];
      }
#pragma unroll
    for (int e = 0; e < kVec; ++e)
      out[(size_t)row_out * W + c + e] = from_f32<TO>(u[e] * r * (w_offset + load_as_f32(norm_w, nw_dtype, c + e)));
  }
}

template <typename T>
__global__ void hyper_fanout_kernel(float* __restrict__ X, const T* __restrict__ h, int S, int W, size_t n) {
  pdl_start();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / W, c = i - t * W;
    const float v = to_f32(h[i]);
    for (int s = 0; s < S; ++s) X[(t * S + s) * W + c] = v;
  }
}

__global__ void scaled_sum_kernel(float* __restrict__ out, const float* __restrict__ a, const float* __restrict__ b, float ca,
                                  float cb, size_t n) {
  pdl_start();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = ca * a[i] + cb * b[i];
}

int blocks_for(size_t n) { return (int)((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256); }

}  // namespace

OI_API int oi_hyper_step(float* X, int rows, int S, int W, const float* y, const float* y2, float c1, float c2, const void* mix,
                         const void* b_out, const void* a_in, int p_dtype, const void* norm_w, int nw_dtype, float eps,
                         float w_offset, void* out, int out_dtype, const int* row_idx, void* stream) {
  OI_REQUIRE(rows >= 0 && S >= 1 && S <= kStreamLimit && W > 0, "hyper_step: bad sizes rows=%d streams=%d (at most %d) width=%d", rows,
             S, kStreamLimit, W);
  OI_REQUIRE(y != nullptr || out != nullptr, "hyper_step: nothing to do");
  OI_REQUIRE(row_idx == nullptr || y == nullptr, "hyper_step: rows are gathered for reading only");
  OI_REQUIRE(out == nullptr || norm_w != nullptr, "hyper_step: the norm needs its weight");
  if (rows == 0) return OI_OK;
  const bool vec = W % 4 == 0 && (uintptr_t)X % 16 == 0 && (y == nullptr || (uintptr_t)y % 16 == 0) && (y2 == nullptr || (uintptr_t)y2 % 16 == 0);
  const int cols = vec ? W / 4 : W;
  const int threads = (cols >= 1024 || S > 8) ? 256 : (cols >= 256 ? 128 : 64);      // at least S * S threads
  cudaStream_t s = (cudaStream_t)stream;
#define OI_HYPER_S(TO, VEC, MAXS)                                                                                          \
  oi_launch(hyper_step_kernel<TO, VEC, MAXS>, rows, threads, 0, s, X, S, W, y, y2, c1, c2, mix, b_out, a_in, p_dtype, norm_w,     \
            nw_dtype, eps, w_offset, (TO*)out, row_idx)
#define OI_HYPER(TO, VEC)                    \
  do {                                       \
    if (S <= 4) OI_HYPER_S(TO, VEC, 4);      \
    else if (S <= 8) OI_HYPER_S(TO, VEC, 8); \
    else OI_HYPER_S(TO, VEC, 16);            \
  } while (0)
  if (out_dtype == OI_BF16 && out != nullptr) {
    if (vec) OI_HYPER(bf16, 4);
    else OI_HYPER(bf16, 1);
  } else {
    if (vec) OI_HYPER(float, 4);
    else OI_HYPER(float, 1);
  }
#undef OI_HYPER
#undef OI_HYPER_S
  OI_CHECK_LAUNCH();
  return OI_OK;
}

OI_API int oi_hyper_fanout(float* X, const void* h, int h_dtype, int rows, int S, int W, void* stream) {
  OI_REQUIRE(rows >= 0 && S >= 1 && W > 0, "hyper_fanout: bad sizes");
  if (rows == 0) return OI_OK;
  const size_t n = (size_t)rows * W;
  cudaStream_t s = (cudaStream_t)stream;
  if (h_dtype == OI_F32) oi_launch(hyper_fanout_kernel<float>, blocks_for(n), 256, 0, s, X, (const float*)h, S, W, n);
  else if (h_dtype == OI_BF16) oi_launch(hyper_fanout_kernel<bf16>, blocks_for(n), 256, 0, s, X, (const bf16*)h, S, W, n);
  else OI_REQUIRE(false, "hyper_fanout: unknown dtype code %d", h_dtype);
  OI_CHECK_LAUNCH();
  return OI_OK;
}

OI_API int oi_scaled_sum(float* out, const float* a, const float* b, float ca, float cb, long long n, void* stream) {
  OI_REQUIRE(n >= 0, "scaled_sum: bad size");
  if (n == 0) return OI_OK;
  oi_launch(scaled_sum_kernel, blocks_for((size_t)n), 256, 0, (cudaStream_t)stream, out, a, b, ca, cb, (size_t)n);
  OI_CHECK_LAUNCH();
  return OI_OK;
}
