// Row and channel steps of layers that keep their residual stream in 32-bit while the products run in the
// model's type: a norm that reads one type and writes another, the norm on a branch's OUTPUT fused with the
// residual sum (and with a weighted average over the outputs of all earlier layers), a short causal
// convolution over time with a per-request state, the norm + page write of a latent that attention reads
// as keys and values alike, a sigmoid gate per head, and the xIELU activation.
//
// All arithmetic is float32 with one rounding at the output. None of these kernels depends on how a
// request's tokens were cut into steps: rows are independent, and the convolution takes the inputs that lie
// before a portion from the request's state.
#include "oi_api.h"

namespace {

constexpr int kRowThreads = 256;

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
// log(1 + e^x) without overflow
__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

// ---------------------------------------------------------------------------------------------
// out[r] = round( x[src] * rsqrt(mean(x[src]^2) + eps) * (w_offset + w) ), src = row_idx ? row_idx[r] : r
// ---------------------------------------------------------------------------------------------
template <typename TX, typename TO>
__global__ void rmsnorm_cast_kernel(TO* __restrict__ out, const TX* __restrict__ x, const void* __restrict__ w, int w_dtype,
                                    const int* __restrict__ row_idx, int hidden, float eps, float w_offset) {
  pdl_start();
  __shared__ float red[32];
  const int r = blockIdx.x;
  const size_t src = row_idx ? (size_t)row_idx[r] : (size_t)r;
  const TX* xr = x + src * hidden;
  float ss = 0.f;
  for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
    const float v = to_f32(xr[d]);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  TO* o = out + (size_t)r * hidden;
  for (int d = threadIdx.x; d < hidden; d += blockDim.x)
    o[d] = from_f32<TO>(to_f32(xr[d]) * inv * (w_offset + load_as_f32(w, w_dtype, d)));
}

// ---------------------------------------------------------------------------------------------
// v = h[r] + a[r] * rsqrt(mean(a[r]^2) + eps) * (w_offset + w)         (the branch's output, normed, joins the stream)
// without history:  h[r] = v
// with history:     hist[n_prev][r] = v;  h[r] = sum_{j < n_prev} coef[j] * hist[j][r] + coef[n_prev] * v
// low != null:      low[r] = round(h[r]) in bfloat16, for the product that reads the stream next
// ---------------------------------------------------------------------------------------------
template <typename TA>
__global__ void branch_norm_add_kernel(float* __restrict__ h, const TA* __restrict__ a, const void* __restrict__ w, int w_dtype,
                                       int hidden, float eps, float w_offset, float* __restrict__ hist, long long hist_stride,
                                       int n_prev, const void* __restrict__ coef, int coef_dtype, bf16* __restrict__ low) {
  pdl_start();
  __shared__ float red[32];
  const size_t row = (size_t)blockIdx.x * hidden;
  const TA* ar = a + row;
  float ss = 0.f;
  for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
    const float v = to_f32(ar[d]);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
    const float v = h[row + d] + to_f32(ar[d]) * inv * (w_offset + load_as_f32(w, w_dtype, d));
    float next = v;
    if (hist != nullptr) {
      hist[(size_t)n_prev * hist_stride + row + d] = v;
      float acc = 0.f;
      for (int j = 0; j < n_prev; ++j) acc += load_as_f32(coef, coef_dtype, j) * hist[(size_t)j * hist_stride + row + d];
      next = acc + load_as_f32(coef, coef_dtype, n_prev) * v;
    }
    h[row + d] = next;
    if (low != nullptr) low[row + d] = __float2bfloat16_rn(next);
  }
}

// the average alone (a layer without any branch norm in front of it): hist[n_prev] = h, h = sum_j coef[j] hist[j]
__global__ void history_average_kernel(float* __restrict__ h, float* __restrict__ hist, long long hist_stride, int n_prev,
                                       const void* __restrict__ coef, int coef_dtype, long long n) {
  pdl_start();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = h[i];
    hist[(size_t)n_prev * hist_stride + i] = v;
    float acc = 0.f;
    for (int j = 0; j < n_prev; ++j) acc += load_as_f32(coef, coef_dtype, j) * hist[(size_t)j * hist_stride + i];
    h[i] = acc + load_as_f32(coef, coef_dtype, n_prev) * v;
  }
}

// ---------------------------------------------------------------------------------------------
// out[t, c] = x[t, c] + sum_{j < taps} w[c, j] * x_(t - taps + 1 + j)[c]: inputs before the portion's first row come
// from the request's state (the last taps - 1 inputs of earlier steps, zeros before the sequence's start).
// ---------------------------------------------------------------------------------------------
template <typename TX, typename TO>
__global__ void short_conv_kernel(TO* __restrict__ out, const TX* __restrict__ x, const void* __restrict__ w, int w_dtype,
                                  const float* __restrict__ state, long long state_stride, const int* __restrict__ cu_seqlens,
                                  const int* __restrict__ token_req, const int* __restrict__ state_slots, int channels,
                                  int taps, int add_input) {
  pdl_start();
  const int t = blockIdx.x;
  const int req = token_req[t];
  const int start = req >= 0 ? cu_seqlens[req] : t;
  const int rel = t - start;
  const float* st = req >= 0 ? state + (size_t)state_slots[req] * state_stride : nullptr;
  const int keep = taps - 1;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
    const float cur = to_f32(x[(size_t)t * channels + c]);
    float acc = add_input ? cur : 0.f;
    for (int j = 0; j < taps; ++j) {
      const int s = rel - keep + j;
      float v;
      if (s >= 0)
        v = to_f32(x[(size_t)(start + s) * channels + c]);
      else
        v = st ? st[(size_t)(keep + s) * channels + c] : 0.f;
      acc += load_as_f32(w, w_dtype, (size_t)c * taps + j) * v;
    }
    out[(size_t)t * channels + c] = from_f32<TO>(acc);
  }
}

// state <- the last taps - 1 inputs of (state, this step's rows), per request and channel
template <typename TX>
__global__ void short_conv_state_kernel(float* __restrict__ state, long long state_stride, const TX* __restrict__ x,
                                        const int* __restrict__ cu_seqlens, const int* __restrict__ token_req,
                                        const int* __restrict__ state_slots, int channels, int keep) {
  pdl_start();
  const int b = blockIdx.x;
  const int start = cu_seqlens[b], n = cu_seqlens[b + 1] - start;
  if (n <= 0 || token_req[start] < 0) return;   // a padding request of a recorded step owns no state
  float* st = state + (size_t)state_slots[b] * state_stride;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
    for (int k = 0; k < keep; ++k) {   // ascending: entry k takes what lies n places further on, or a row of the step
      const int s = n + k - keep;
      st[(size_t)k * channels + c] = s >= 0 ? to_f32(x[(size_t)(start + s) * channels + c]) : st[(size_t)(k + n) * channels + c];
    }
  }
}

// ---------------------------------------------------------------------------------------------
// latent[t] = round( z * rsqrt(mean(z^2) + eps) * (w_offset + w) ), z = src[t, 0..rank), stored at the row's slot of
// the pages (rows of `row_elems` >= rank elements, the rest zero)
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void latent_store_kernel(T* __restrict__ pages, long long page_stride, int page_size, int row_elems,
                                    const T* __restrict__ src, long long src_stride, const void* __restrict__ w, int w_dtype,
                                    const int* __restrict__ slots, int rank, float eps, float w_offset) {
  pdl_start();
  __shared__ float red[32];
  const int t = blockIdx.x;
  const int slot = slots[t];
  if (slot < 0) return;     // whole block leaves
  const T* z = src + (size_t)t * src_stride;
  float ss = 0.f;
  for (int d = threadIdx.x; d < rank; d += blockDim.x) {
    const float v = to_f32(z[d]);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)rank + eps);
  T* dst = pages + (size_t)(slot / page_size) * page_stride + (size_t)(slot % page_size) * row_elems;
  for (int d = threadIdx.x; d < row_elems; d += blockDim.x)
    dst[d] = d < rank ? from_f32<T>(to_f32(z[d]) * inv * (w_offset + load_as_f32(w, w_dtype, d))) : from_f32<T>(0.f);
}

// o[t, h, :] *= sigmoid(g[t, h])
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ o, long long o_stride, const T* __restrict__ g, long long g_stride, int heads,
                                 int head_elems, long long n) {
  pdl_start();
  const int per_row = heads * head_elems;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / per_row;
    const int r = (int)(i - t * per_row);
    const float gate = sigmoid_f(to_f32(g[t * g_stride + r / head_elems]));
    T* p = o + t * o_stride + r;
    *p = from_f32<T>(to_f32(*p) * gate);
  }
}

// xIELU with learned shape: z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z / 2
template <typename T>
__global__ void xielu_kernel(T* out, const T* in, const void* __restrict__ pq, int pq_dtype, long long n) {
  pdl_start();
  const float ap = softplus_f(load_as_f32(pq, pq_dtype, 0));
  const float an = 0.5f + softplus_f(load_as_f32(pq, pq_dtype, 1));
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float z = to_f32(in[i]);
    const float v = z > 0.f ? ap * z * z + 0.5f * z : an * (expm1f(z) - z) + 0.5f * z;
    out[i] = from_f32<T>(v);
  }
}

int flat_blocks(long long n) {
  const long long b = (n + kRowThreads - 1) / kRowThreads;
  return (int)(b > 148 * 16 ? 148 * 16 : (b < 1 ? 1 : b));
}

}  // namespace

OI_API int oi_rmsnorm_cast(void* out, int out_dtype, const void* x, int x_dtype, const void* w, int w_dtype, const int* row_idx,
                           int rows, int hidden, float eps, float w_offset, void* stream) {
  OI_REQUIRE(rows >= 0 && hidden > 0, "rmsnorm_cast: bad sizes rows=%d hidden=%d", rows, hidden);
  if (rows == 0) return OI_OK;
  cudaStream_t s = (cudaStream_t)stream;
#define OI_CAST_CASE(XD, OD, TX, TO)                                                                                  \
  if (x_dtype == XD && out_dtype == OD) {                                                                             \
    oi_launch(rmsnorm_cast_kernel<TX, TO>, rows, kRowThreads, 0, s, (TO*)out, (const TX*)x, w, w_dtype, row_idx, hidden, eps, \
              w_offset);                                                                                              \
    OI_CHECK_LAUNCH();                                                                                                \
    return OI_OK;                                                                                                     \
  }
  OI_CAST_CASE(OI_F32, OI_F32, float, float)
  OI_CAST_CASE(OI_F32, OI_BF16, float, bf16)
  OI_CAST_CASE(OI_BF16, OI_F32, bf16, float)
  OI_CAST_CASE(OI_BF16, OI_BF16, bf16, bf16)
#undef OI_CAST_CASE
  OI_REQUIRE(false, "rmsnorm_cast: unknown dtype codes %d -> %d", x_dtype, out_dtype);
}

OI_API int oi_branch_norm_add(float* h, const void* a, int a_dtype, const void* w, int w_dtype, int rows, int hidden, float eps,
                              float w_offset, float* hist, long long hist_stride, int n_prev, const void* coef, int coef_dtype,
                              void* low, void* stream) {
  OI_REQUIRE(rows >= 0 && hidden > 0, "branch_norm_add: bad sizes rows=%d hidden=%d", rows, hidden);
  OI_REQUIRE(hist == nullptr || (coef != nullptr && n_prev >= 0 && hist_stride >= (long long)rows * hidden),
             "branch_norm_add: the history needs coefficients and a stride of at least rows * hidden");
  if (rows == 0) return OI_OK;
  cudaStream_t s = (cudaStream_t)stream;
  if (a_dtype == OI_F32)
    oi_launch(branch_norm_add_kernel<float>, rows, kRowThreads, 0, s, h, (const float*)a, w, w_dtype, hidden, eps, w_offset, hist,
              hist_stride, n_prev, coef, coef_dtype, (bf16*)low);
  else if (a_dtype == OI_BF16)
    oi_launch(branch_norm_add_kernel<bf16>, rows, kRowThreads, 0, s, h, (const bf16*)a, w, w_dtype, hidden, eps, w_offset, hist,
              hist_stride, n_prev, coef, coef_dtype, (bf16*)low);
  else
    OI_REQUIRE(false, "branch_norm_add: unknown dtype code %d", a_dtype);
  OI_CHECK_LAUNCH();
  return OI_OK;
}

OI_API int oi_history_average(float* h, float* hist, long long hist_stride, int n_prev, const void* coef, int coef_dtype,
                              long long n, void* stream) {
  OI_REQUIRE(h && hist && coef && n_prev >= 0 && n >= 0 && hist_stride >= n, "history_average: bad arguments");
  if (n == 0) return OI_OK;
  oi_launch(history_average_kernel, flat_blocks(n), kRowThreads, 0, (cudaStream_t)stream, h, hist, hist_stride, n_prev, coef,
            coef_dtype, n);
  OI_CHECK_LAUNCH();
  return OI_OK;
}

OI_API int oi_short_conv(void* out, int out_dtype, const void* x, int x_dtype, const void* w, int w_dtype, float* state,
                         long long state_stride, const int* cu_seqlens, const int* token_req, const int* state_slots, int tokens,
                         int requests, int channels, int taps, int add_input, int update_state, void* stream) {
  OI_REQUIRE(tokens >= 0 && requests >= 0 && channels > 0 && taps >= 1, "short_conv: bad sizes tokens=%d channels=%d taps=%d",
             tokens, channels, taps);
  OI_REQUIRE(taps == 1 || (state != nullptr && state_stride >= (long long)(taps - 1) * channels),
             "short_conv: %d taps need a state of %d rows per request", taps, taps - 1);
  if (tokens == 0) return OI_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int cy = (channels + kRowThreads - 1) / kRowThreads;
  const dim3 grid(tokens, cy);
#define OI_CONV_CASE(XD, OD, TX, TO)                                                                                     \
  if (x_dtype == XD && out_dtype == OD) {                                                                                \
    oi_launch(short_conv_kernel<TX, TO>, grid, kRowThreads, 0, s, (TO*)out, (const TX*)x, w, w_dtype, (const float*)state, \
              state_stride, cu_seqlens, token_req, state_slots, channels, taps, add_input);                              \
    OI_CHECK_LAUNCH();                                                                                                   \
    if (update_state && taps > 1) {                                                                                      \
      oi_launch(short_conv_state_kernel<TX>, dim3(requests, cy), kRowThreads, 0, s, state, state_stride, (const TX*)x,    \
                cu_seqlens, token_req, state_slots, channels, taps - 1);                                                 \
      OI_CHECK_LAUNCH();                                                                                                 \
    }                                                                                                                    \
    return OI_OK;                                                                                                        \
  }
  OI_CONV_CASE(OI_F32, OI_F32, float, float)
  OI_CONV_CASE(OI_F32, OI_BF16, float, bf16)
  OI_CONV_CASE(OI_BF16, OI_BF16, bf16, bf16)
#undef OI_CONV_CASE
  OI_REQUIRE(false, "short_conv: dtype codes %d -> %d are not supported", x_dtype, out_dtype);
}

OI_API int oi_latent_store(void* pages, long long page_stride, int page_size, int row_elems, const void* src, long long src_stride,
                           int dtype, const void* w, int w_dtype, const int* slots, int tokens, int rank, float eps, float w_offset,
                           void* stream) {
  OI_REQUIRE(tokens >= 0 && rank > 0 && row_elems >= rank && page_size > 0, "latent_store: bad sizes rank=%d row=%d", rank, row_elems);
  if (tokens == 0) return OI_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = rank <= 64 ? 64 : (rank <= 128 ? 128 : kRowThreads);
  if (dtype == OI_F32)
    oi_launch(latent_store_kernel<float>, tokens, threads, 0, s, (float*)pages, page_stride, page_size, row_elems, (const float*)src,
              src_stride, w, w_dtype, slots, rank, eps, w_offset);
  else if (dtype == OI_BF16)
    oi_launch(latent_store_kernel<bf16>, tokens, threads, 0, s, (bf16*)pages, page_stride, page_size, row_elems, (const bf16*)src,
              src_stride, w, w_dtype, slots, rank, eps, w_offset);
  else
    OI_REQUIRE(false, "latent_store: unknown dtype code %d", dtype);
  OI_CHECK_LAUNCH();
  return OI_OK;
}

OI_API int oi_head_gate(void* o, long long o_stride, const void* g, long long g_stride, int dtype, int tokens, int heads,
                        int head_elems, void* stream) {
  OI_REQUIRE(tokens >= 0 && heads > 0 && head_elems > 0, "head_gate: bad sizes");
  const long long n = (long long)tokens * heads * head_elems;
  if (n == 0) return OI_OK;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == OI_F32)
    oi_launch(head_gate_kernel<float>, flat_blocks(n), kRowThreads, 0, s, (float*)o, o_stride, (const float*)g, g_stride, heads,
              head_elems, n);
  else if (dtype == OI_BF16)
    oi_launch(head_gate_kernel<bf16>, flat_blocks(n), kRowThreads, 0, s, (bf16*)o, o_stride, (const bf16*)g, g_stride, heads,
              head_elems, n);
  else
    OI_REQUIRE(false, "head_gate: unknown dtype code %d", dtype);
  OI_CHECK_LAUNCH();
  return OI_OK;
}

OI_API int oi_xielu(void* out, const void* in, int dtype, const void* pq, int pq_dtype, long long n, void* stream) {
  OI_REQUIRE(n >= 0 && pq != nullptr, "xielu: bad arguments");
  if (n == 0) return OI_OK;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == OI_F32)
    oi_launch(xielu_kernel<float>, flat_blocks(n), kRowThreads, 0, s, (float*)out, (const float*)in, pq, pq_dtype, n);
  else if (dtype == OI_BF16)
    oi_launch(xielu_kernel<bf16>, flat_blocks(n), kRowThreads, 0, s, (bf16*)out, (const bf16*)in, pq, pq_dtype, n);
  else
    OI_REQUIRE(false, "xielu: unknown dtype code %d", dtype);
  OI_CHECK_LAUNCH();
  return OI_OK;
}
