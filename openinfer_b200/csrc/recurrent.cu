// Recurrent mixers whose memory is a matrix per head: a scan over the rows of a step, request by request.
//
// Both kinds keep, per request and head, C [D keys x V values] in float32 and update it token by token:
//
//   kMatrixMemory (the mLSTM cell):  m' = max(f + m, i);  C' = e^(f + m - m') C + e^(i - m') k v^T;  n' likewise with k;
//                                    o = C'^T q / (max(|n' . q|, e^(-m')) + 1e-6);  i = cap tanh(zi / cap),
//                                    f = logsigmoid(cap tanh(zf / cap)); q arrives unscaled and is multiplied by q_scale
//   kGatedDelta (gated delta rule):  C <- diag(g) C;  d = beta (v - C^T k);  C <- C + k d^T;  o = C^T q, with k and q made
//                                    unit vectors (1e-6 inside the root), q times q_scale, beta = sigmoid(zb) and one decay
//                                    per key channel g = exp(-exp(A_h) softplus(a + dt))
//
// One launch serves prompts and single decoded tokens alike: block (request, head, slice of 8 value columns) walks the
// request's rows of the step in order, the state in registers (a column's D numbers spread over 16 lanes), the next row's
// inputs requested while the current one is worked on. The state lives in two copies that take turns ([slots][2][heads]
// [elems], C stored column by column, then n and m): a step reads copy state_phase[request] and leaves the other, so no
// block reads what another writes. Everything is float32: the inputs are the float32 sums of the projections.
#include "common.cuh"

namespace {

constexpr int kLanes = 16;     // lanes that share a value column
constexpr int kCols = 8;       // value columns per block
enum : int { kMatrixMemory = 0, kGatedDelta = 1 };

struct ScanArgs {
  const float* qkv;            // [tokens, ld_qkv]: queries, keys (kv head major, D each) and values (head major, V each)
  long long ld_qkv;
  int q_off, k_off, v_off;
  const float* gates;          // [tokens, ld_gates]: matrix memory: zi at i_off + h, zf at f_off + h; delta: zb at i_off + h
  long long ld_gates;
  int i_off, f_off;
  const float* decay;          // delta: a [tokens, ld_decay], head major, D each
  long long ld_decay;
  const void* p0;              // matrix memory: bias of zi [H]; delta: dt [H * D]
  const void* p1;              // matrix memory: bias of zf [H]; delta: A [H]
  int p_dtype;
  float cap, q_scale;
  float* state;
  long long state_stride;      // floats between slots (two copies inside)
  const int* cu_seqlens;
  const int* token_req;
  const int* state_slots;
  const int* state_phase;
  float* out;                  // [tokens, ld_out], head major, V each
  long long ld_out;
  int H, G, D, V;
};

__device__ __forceinline__ float lanes_sum(float v) {
#pragma unroll
  for (int o = kLanes / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

template <int kMode, int R>
__global__ void __launch_bounds__(kLanes* kCols) recurrent_scan_kernel(ScanArgs a) {
  pdl_start();
  const int b = blockIdx.x, h = blockIdx.y;
  const int start = a.cu_seqlens[b], n_rows = a.cu_seqlens[b + 1] - start;
  if (n_rows <= 0 || a.token_req[start] < 0) return;    // a padding request of a recorded step owns no state
  const int j = threadIdx.x % kLanes;
  const int c = blockIdx.z * kCols + threadIdx.x / kLanes;
  const bool col = c < a.V;
  const int D = a.D, V = a.V;
  const int g = h / (a.H / a.G);
  const int elems = D * V + (kMode == kMatrixMemory ? D + 1 : 0);
  const int phase = a.state_phase[b];
  const float* old = a.state + (size_t)a.state_slots[b] * a.state_stride + ((size_t)phase * a.H + h) * elems;
  float* fresh = a.state + (size_t)a.state_slots[b] * a.state_stride + ((size_t)(1 - phase) * a.H + h) * elems;

  float C[R], nn[R], par[R];   // par: delta: dt of the thread's channels
  float m = 0.f, p1 = 0.f, p0 = 0.f;
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int d = j + i * kLanes;
    C[i] = (col && d < D) ? old[(size_t)c * D + d] : 0.f;
    nn[i] = 0.f;
    par[i] = 0.f;
    if (kMode == kMatrixMemory && d < D) nn[i] = old[(size_t)D * V + d];
    if (kMode == kGatedDelta && d < D) par[i] = load_as_f32(a.p0, a.p_dtype, (size_t)h * D + d);
  }
  if (kMode == kMatrixMemory) {
    m = old[(size_t)D * V + D];
    p0 = load_as_f32(a.p0, a.p_dtype, h);
    p1 = load_as_f32(a.p1, a.p_dtype, h);
  } else {
    p1 = expf(load_as_f32(a.p1, a.p_dtype, h));
  }

  // the next row's inputs, requested one row ahead
  float kq[R], qq[R], aa[R], vv = 0.f, z0 = 0.f, z1 = 0.f;
  auto fetch = [&](int row) {
    const float* r = a.qkv + (size_t)row * a.ld_qkv;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int d = j + i * kLanes;
      kq[i] = d < D ? r[a.k_off + g * D + d] : 0.f;
      qq[i] = d < D ? r[a.q_off + g * D + d] : 0.f;
      if (kMode == kGatedDelta) aa[i] = d < D ? a.decay[(size_t)row * a.ld_decay + (size_t)h * D + d] : 0.f;
    }
    vv = col ? r[a.v_off + h * V + c] : 0.f;
    const float* gr = a.gates + (size_t)row * a.ld_gates;
    z0 = gr[a.i_off + h];
    if (kMode == kMatrixMemory) z1 = gr[a.f_off + h];
  };
  fetch(start);
  for (int t = 0; t < n_rows; ++t) {
    float k[R], q[R], dec[R];
    const float v = vv, zi = z0, zf = z1;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      k[i] = kq[i];
      q[i] = qq[i];
      if (kMode == kGatedDelta) dec[i] = aa[i];
    }
    if (t + 1 < n_rows) fetch(start + t + 1);
    float o;
    if (kMode == kMatrixMemory) {
      const float gi = a.cap * tanhf((zi + p0) / a.cap);
      const float fx = a.cap * tanhf((zf + p1) / a.cap);
      const float gf = fminf(fx, 0.f) - log1pf(expf(-fabsf(fx)));     // logsigmoid
      const float m_new = fmaxf(gf + m, gi);
      const float keep = expf(gf + m - m_new), put = expf(gi - m_new);
      m = m_new;
      float num = 0.f, nq = 0.f;
#pragma unroll
      for (int i = 0; i < R; ++i) {
        const float qs = q[i] * a.q_scale;
        C[i] = keep * C[i] + put * k[i] * v;
        nn[i] = keep * nn[i] + put * k[i];
        num += C[i] * qs;
        nq += nn[i] * qs;
      }
      num = lanes_sum(num);
      nq = lanes_sum(nq);
      o = num / (fmaxf(fabsf(nq), expf(-m)) + 1e-6f);
    } else {
      float k2 = 0.f, q2 = 0.f;
#pragma unroll
      for (int i = 0; i < R; ++i) {
        k2 += k[i] * k[i];
        q2 += q[i] * q[i];
      }
      k2 = lanes_sum(k2);
      q2 = lanes_sum(q2);
      const float kn = 1.f / sqrtf(k2 + 1e-6f), qn = a.q_scale / sqrtf(q2 + 1e-6f);
      const float beta = 1.f / (1.f + expf(-zi));
      float kv = 0.f;
#pragma unroll
      for (int i = 0; i < R; ++i) {
        k[i] *= kn;
        C[i] *= expf(-p1 * softplus_f(dec[i] + par[i]));
        kv += C[i] * k[i];
      }
      kv = lanes_sum(kv);
      const float d = beta * (v - kv);
      float num = 0.f;
#pragma unroll
      for (int i = 0; i < R; ++i) {
        C[i] += k[i] * d;
        num += C[i] * (q[i] * qn);
      }
      o = lanes_sum(num);
    }
    if (j == 0 && col) a.out[(size_t)(start + t) * a.ld_out + (size_t)h * V + c] = o;
  }
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int d = j + i * kLanes;
    if (col && d < D) fresh[(size_t)c * D + d] = C[i];
    if (kMode == kMatrixMemory && blockIdx.z == 0 && threadIdx.x < kLanes && d < D) fresh[(size_t)D * V + d] = nn[i];
  }
  if (kMode == kMatrixMemory && blockIdx.z == 0 && threadIdx.x == 0) fresh[(size_t)D * V + D] = m;
}

// out[t, h, c] = o[t, h, c] * rsqrt(mean_c o[t, h, :]^2 + eps) * w[h * w_stride + c] * sigmoid(gate[t, h, c]) * scale:
// the per-head unit norm, the weight and the output gate of a recurrent mixer, one warp per (row, head).
template <typename TO>
__global__ void head_norm_gate_kernel(TO* __restrict__ out, long long ld_out, const float* __restrict__ o, long long ld_o,
                                      const float* __restrict__ gate, long long ld_gate, const void* __restrict__ w,
                                      int w_dtype, int w_stride, int tokens, int H, int V, float eps, float scale) {
  pdl_start();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= tokens * H) return;
  const int t = warp / H, h = warp - t * H;
  const float* row = o + (size_t)t * ld_o + (size_t)h * V;
  float ss = 0.f;
  for (int c = lane; c < V; c += 32) ss += row[c] * row[c];
  ss = warp_sum(ss);
  const float r = 1.f / sqrtf(ss / (float)V + eps);
  for (int c = lane; c < V; c += 32) {
    const float gz = gate[(size_t)t * ld_gate + (size_t)h * V + c];
    const float val = row[c] * r * load_as_f32(w, w_dtype, (size_t)h * w_stride + c) * (1.f / (1.f + expf(-gz))) * scale;
    out[(size_t)t * ld_out + (size_t)h * V + c] = from_f32<TO>(val);
  }
}

}  // namespace

// mode 0: matrix memory (p0, p1: the two gate biases [H]); mode 1: gated delta rule (p0: dt [H * D], p1: A [H];
// decay: a [tokens, ld_decay]). State: [slots][2][H][D * V (+ D + 1 in mode 0)] floats.
OI_API int oi_recurrent_scan(int mode, const float* qkv, long long ld_qkv, int q_off, int k_off, int v_off, const float* gates,
                             long long ld_gates, int i_off, int f_off, const float* decay, long long ld_decay, const void* p0,
                             const void* p1, int p_dtype, float cap, float q_scale, float* state, long long state_stride,
                             const int* cu_seqlens, const int* token_req, const int* state_slots, const int* state_phase,
                             float* out, long long ld_out, int requests, int H, int G, int D, int V, void* stream) {
  OI_REQUIRE(mode == kMatrixMemory || mode == kGatedDelta, "recurrent_scan: unknown mode %d", mode);
  OI_REQUIRE(requests >= 0 && H > 0 && G > 0 && H % G == 0 && D > 0 && V > 0, "recurrent_scan: bad sizes H=%d G=%d D=%d V=%d", H, G, D, V);
  OI_REQUIRE(D <= 16 * kLanes, "recurrent_scan: %d key channels per head, at most %d", D, 16 * kLanes);
  OI_REQUIRE(mode != kGatedDelta || decay != nullptr, "recurrent_scan: the delta rule needs its decays");
  const long long elems = (long long)D * V + (mode == kMatrixMemory ? D + 1 : 0);
  OI_REQUIRE(state != nullptr && state_stride >= 2 * H * elems, "recurrent_scan: the state needs two copies of %lld floats per head", elems);
  if (requests == 0) return OI_OK;
  ScanArgs a;
  a.qkv = qkv, a.ld_qkv = ld_qkv, a.q_off = q_off, a.k_off = k_off, a.v_off = v_off;
  a.gates = gates, a.ld_gates = ld_gates, a.i_off = i_off, a.f_off = f_off;
  a.decay = decay, a.ld_decay = ld_decay, a.p0 = p0, a.p1 = p1, a.p_dtype = p_dtype, a.cap = cap, a.q_scale = q_scale;
  a.state = state, a.state_stride = state_stride, a.cu_seqlens = cu_seqlens, a.token_req = token_req;
  a.state_slots = state_slots, a.state_phase = state_phase, a.out = out, a.ld_out = ld_out;
  a.H = H, a.G = G, a.D = D, a.V = V;
  const dim3 grid(requests, H, (V + kCols - 1) / kCols);
  cudaStream_t s = (cudaStream_t)stream;
  const int r = (D + kLanes - 1) / kLanes;
#define OI_SCAN(MODE)                                                                                         \
  do {                                                                                                        \
    if (r <= 4) oi_launch(recurrent_scan_kernel<MODE, 4>, grid, kLanes * kCols, 0, s, a);                     \
    else if (r <= 8) oi_launch(recurrent_scan_kernel<MODE, 8>, grid, kLanes * kCols, 0, s, a);                \
    else oi_launch(recurrent_scan_kernel<MODE, 16>, grid, kLanes * kCols, 0, s, a);                           \
  } while (0)
  if (mode == kMatrixMemory) OI_SCAN(kMatrixMemory);
  else OI_SCAN(kGatedDelta);
#undef OI_SCAN
  OI_CHECK_LAUNCH();
  return OI_OK;
}

OI_API int oi_head_norm_gate(void* out, int out_dtype, long long ld_out, const float* o, long long ld_o, const float* gate,
                             long long ld_gate, const void* w, int w_dtype, int w_stride, int tokens, int H, int V, float eps,
                             float scale, void* stream) {
  OI_REQUIRE(tokens >= 0 && H > 0 && V > 0, "head_norm_gate: bad sizes");
  if (tokens == 0) return OI_OK;
  const int warps = tokens * H, blocks = (warps + 7) / 8;
  cudaStream_t s = (cudaStream_t)stream;
  if (out_dtype == OI_F32)
    oi_launch(head_norm_gate_kernel<float>, blocks, 256, 0, s, (float*)out, ld_out, o, ld_o, gate, ld_gate, w, w_dtype, w_stride, tokens, H, V, eps, scale);
  else if (out_dtype == OI_BF16)
    oi_launch(head_norm_gate_kernel<bf16>, blocks, 256, 0, s, (bf16*)out, ld_out, o, ld_o, gate, ld_gate, w, w_dtype, w_stride, tokens, H, V, eps, scale);
  else
    OI_REQUIRE(false, "head_norm_gate: unknown dtype code %d", out_dtype);
  OI_CHECK_LAUNCH();
  return OI_OK;
}
