// Generalized delta rule: a recurrent mixer whose state per head is a matrix S [key channel,
// value channel] in 32-bit floats, carried from token to token:
//
//   S <- diag(w) S  -  (a * u) (u^T S)  +  k v^T          (both products read the old S)
//   o  = S^T r
//
// with per-channel decay w = exp(-rate * sigmoid(d)), removal rate a = sigmoid(.), and the unit key
// u = k / sqrt(sum k^2 + 1e-6).  The kernel takes the projections r, k, v, the gate's and the two
// rates' pre-activations in 32-bit, forms every quantity of the recurrence in 32-bit, walks a
// request's tokens in order, divides each head's o by its root mean square, multiplies by a weight
// and by sigmoid(gate) and rounds to the storage type for the output projection.
//
// One CTA per (head, request).  Built per head size D (LAB_HEAD_DIM).  The columns of S are
// independent of one another, so thread (j, g) keeps rows g*SL .. g*SL+SL-1 of column j in
// registers (G = 4 threads per column, sums over rows finished with two shuffles).  Tokens are
// taken in chunks: the chunk's vectors are prepared in shared memory by all threads, then the
// threads walk the chunk's tokens without a block-wide barrier.  A step of one token per request
// (decode) is the same kernel with a chunk of one.
#include "common.cuh"

#ifndef LAB_HEAD_DIM
#define LAB_HEAD_DIM 64
#endif

namespace {

constexpr int D = LAB_HEAD_DIM;
constexpr int G = 4;
constexpr int SL = (D + G - 1) / G;
constexpr int NT = ((D * G + 31) / 32) * 32;
constexpr int CH = D > 128 ? 4 : 8;
static_assert(D >= 4 && D <= 256, "head size of the delta rule kernel: 4 to 256");

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }

struct DeltaParams {
  void* out;            // [tokens, heads * D] of T
  const float* r;       // the five projections: [tokens, ld] floats each
  const float* k;
  const float* v;
  const float* g;
  const float* a;
  int ld;
  const float* d;       // decay pre-activation (before its bias) [tokens, ld_d]
  int ld_d;
  const void* d_bias;   // [heads * D] of T
  const void* a_bias;   // [heads * D] of T
  const void* norm_w;   // [heads * D] of T
  float* state;         // [slots, heads, D, D] floats
  const int* q_start;   // [requests + 1]
  const int* state_slot;
  int heads, n_slots, write;
  float eps, decay_rate;
};

template <typename T>
__global__ void __launch_bounds__(NT) delta_rule_kernel(DeltaParams p) {
  __shared__ float s_r[CH][D], s_k[CH][D], s_u[CH][D], s_au[CH][D], s_w[CH][D], s_v[CH][D], s_g[CH][D], s_o[CH][D];
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.x, req = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = NT / 32;
  const int j = tid / G, g = tid % G;
  const bool live = j < D;
  const int row0 = p.q_start[req], row1 = p.q_start[req + 1];
  const int slot = p.state_slot[req];
  if (slot < 0 || slot >= p.n_slots) {
    if (tid == 0) lab_set_error(LAB_ERR_PAGE_RANGE);
    return;
  }
  float* S_g = p.state + ((size_t)slot * p.heads + h) * D * D;
  float S[SL];
#pragma unroll
  for (int ii = 0; ii < SL; ++ii) {
    const int i = g * SL + ii;
    S[ii] = (live && i < D) ? S_g[(size_t)i * D + j] : 0.f;
  }
  const T* d_bias = (const T*)p.d_bias + h * D;
  const T* a_bias = (const T*)p.a_bias + h * D;
  const T* norm_w = (const T*)p.norm_w + h * D;
  T* out = (T*)p.out;
  const int ld_out = p.heads * D;

  for (int t0 = row0; t0 < row1; t0 += CH) {
    const int n = min(CH, row1 - t0);
    // ---- the chunk's vectors ------------------------------------------------------------
    for (int idx = tid; idx < n * D; idx += NT) {
      const int tok = idx / D, i = idx % D;
      const size_t at = (size_t)(t0 + tok) * p.ld + h * D + i;
      s_r[tok][i] = p.r[at];
      s_k[tok][i] = p.k[at];
      s_v[tok][i] = p.v[at];
      s_g[tok][i] = sigmoidf_(p.g[at]);
      s_au[tok][i] = sigmoidf_(p.a[at] + to_f32(a_bias[i]));
      const float dl = p.d[(size_t)(t0 + tok) * p.ld_d + h * D + i] + to_f32(d_bias[i]);
      s_w[tok][i] = expf(-p.decay_rate * sigmoidf_(dl));
    }
    __syncthreads();
    for (int tok = warp; tok < n; tok += nwarps) {
      float ss = 0.f;
      for (int i = lane; i < D; i += 32) ss += s_k[tok][i] * s_k[tok][i];
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss + 1e-6f);
      for (int i = lane; i < D; i += 32) {
        const float u = s_k[tok][i] * inv;
        s_u[tok][i] = u;
        s_au[tok][i] *= u;
      }
    }
    __syncthreads();
    // ---- the recurrence, token by token ---------------------------------------------------
    for (int tok = 0; tok < n; ++tok) {
      float sa = 0.f;
#pragma unroll
      for (int ii = 0; ii < SL; ++ii) {
        const int i = g * SL + ii;
        if (i < D) sa = fmaf(s_u[tok][i], S[ii], sa);
      }
      sa += __shfl_xor_sync(0xffffffffu, sa, 1);
      sa += __shfl_xor_sync(0xffffffffu, sa, 2);
      const float vj = live ? s_v[tok][j] : 0.f;
      float o = 0.f;
#pragma unroll
      for (int ii = 0; ii < SL; ++ii) {
        const int i = g * SL + ii;
        if (i < D) {
          const float s = fmaf(s_k[tok][i], vj, fmaf(s_w[tok][i], S[ii], -s_au[tok][i] * sa));
          S[ii] = s;
          o = fmaf(s, s_r[tok][i], o);
        }
      }
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      if (live && g == 0) s_o[tok][j] = o;
    }
    __syncthreads();
    // ---- each head's o over its root mean square, weight, gate ------------------------------
    for (int tok = warp; tok < n; tok += nwarps) {
      float ss = 0.f;
      for (int i = lane; i < D; i += 32) ss += s_o[tok][i] * s_o[tok][i];
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss / (float)D + p.eps);
      for (int i = lane; i < D; i += 32)
        out[(size_t)(t0 + tok) * ld_out + h * D + i] =
            from_f32<T>(s_o[tok][i] * inv * to_f32(norm_w[i]) * s_g[tok][i]);
    }
    __syncthreads();
  }
  if (p.write) {
#pragma unroll
    for (int ii = 0; ii < SL; ++ii) {
      const int i = g * SL + ii;
      if (live && i < D) S_g[(size_t)i * D + j] = S[ii];
    }
  }
}

// out (T) [tokens, n] = tanh(x [tokens, ld]) for the low-rank middle of the decay's projection
template <typename T>
__global__ void __launch_bounds__(256) tanh_cast_kernel(T* __restrict__ out, const float* __restrict__ x, long long tokens,
                                                        int n, int ld) {
  pdl_trigger();
  pdl_wait();
  const long long total = tokens * n;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256)
    out[i] = from_f32<T>(tanhf(x[(i / n) * ld + (i % n)]));
}

}  // namespace

LAB_EXPORT int lab_delta_rule_head_dim() { return D; }

LAB_EXPORT int lab_delta_rule(void* out, const float* r, const float* k, const float* v, const float* g,
                              const float* a, int ld, const float* d, int ld_d, const void* d_bias,
                              const void* a_bias, const void* norm_w, float* state, const int* q_start,
                              const int* state_slot, int n_requests, int heads, int n_slots, int write, float eps,
                              float decay_rate, int dtype, cudaStream_t stream) {
  if (n_requests <= 0 || heads <= 0) return 0;
  DeltaParams p;
  p.out = out; p.r = r; p.k = k; p.v = v; p.g = g; p.a = a; p.ld = ld; p.d = d; p.ld_d = ld_d;
  p.d_bias = d_bias; p.a_bias = a_bias; p.norm_w = norm_w; p.state = state; p.q_start = q_start;
  p.state_slot = state_slot; p.heads = heads; p.n_slots = n_slots; p.write = write; p.eps = eps;
  p.decay_rate = decay_rate;
  if (dtype == LAB_F32)
    lab_launch(delta_rule_kernel<float>, dim3(heads, n_requests), dim3(NT), 0, stream, p);
  else
    lab_launch(delta_rule_kernel<__nv_bfloat16>, dim3(heads, n_requests), dim3(NT), 0, stream, p);
  LAB_LAUNCH_CHECK();
}

LAB_EXPORT int lab_tanh_cast(void* out, const float* x, long long tokens, int n, int ld, int dtype,
                             cudaStream_t stream) {
  const long long total = tokens * n;
  if (total <= 0) return 0;
  const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  if (dtype == LAB_F32)
    lab_launch(tanh_cast_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)out, x, tokens, n, ld);
  else
    lab_launch(tanh_cast_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)out, x, tokens, n,
               ld);
  LAB_LAUNCH_CHECK();
}
