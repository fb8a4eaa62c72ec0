// Row-wise steps around a softmax attention whose queries and keys are RMS-normed over the whole
// projection (all heads at once) and whose heads' outputs pass a sigmoid gate:
//
//   qk_norm_store   from the fused 32-bit projection [q | k | v | ...] of a step's rows (whole, or as
//                   split-K partial products summed here in ascending order) plus an optional bias:
//                   q <- q / rms(q) * wq, k <- k / rms(k) * wk, each root mean square over the whole
//                   projection of the row; q rounded to T into [tokens, n_q * HD]; k and v rounded into
//                   the row's slot of the paged cache [pages, n_kv, page_size, HD].  A head is stored HD
//                   wide, HD >= max(D, V): the entries beyond a head's own size are zeros, so that heads
//                   whose key and value sizes differ (or are no multiple of the tensor-core tile) run on
//                   the attention kernels built for heads of HD.  A layer that reads another layer's keys
//                   and values has only the q part.
//   head_gate       out[t, h, i] = attn[t, h, i] * sigmoid(g) * c, g one number per head or per entry,
//                   read from the same projection; the V real entries of each head are packed side by
//                   side and rounded to T for the output projection.
//
// All arithmetic is 32-bit; T says how the weights are stored and how results are rounded.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float sum_splits(const float* __restrict__ p, int splits, long long stride, size_t at) {
  float total = 0.f;
  for (int s0 = 0; s0 < splits; s0 += 8) {
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = s0 + j < splits ? p[(s0 + j) * stride + at] : 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) total += v[j];
  }
  return total;
}

struct QkNormParams {
  const float* proj;
  int splits;
  long long split_stride;
  int ld;
  const int* slots;
  int n_q, n_kv, D, V, HD, page_size, num_pages, has_kv, ld_q;
  float eps;
};

template <typename T>
__global__ void __launch_bounds__(kThreads) qk_norm_store_kernel(T* __restrict__ q_out, T* __restrict__ cache_k,
                                                                 T* __restrict__ cache_v, const T* __restrict__ bias,
                                                                 const T* __restrict__ wq, const T* __restrict__ wk,
                                                                 QkNormParams p) {
  extern __shared__ float row[];      // [n_q * D + n_kv * (D + V)]
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int wq_n = p.n_q * p.D, wk_n = p.has_kv ? p.n_kv * p.D : 0, wv_n = p.has_kv ? p.n_kv * p.V : 0;
  const int total = wq_n + wk_n + wv_n;
  float ssq = 0.f, ssk = 0.f;
  for (int i = threadIdx.x; i < total; i += kThreads) {
    float v = sum_splits(p.proj, p.splits, p.split_stride, (size_t)t * p.ld + i);
    if (bias != nullptr) v += to_f32(bias[i]);
    row[i] = v;
    if (i < wq_n) ssq += v * v;
    else if (i < wq_n + wk_n) ssk += v * v;
  }
  ssq = block_sum(ssq, scratch);
  const float inv_q = 1.0f / sqrtf(ssq / (float)wq_n + p.eps);
  for (int idx = threadIdx.x; idx < p.n_q * p.HD; idx += kThreads) {
    const int h = idx / p.HD, i = idx - h * p.HD;
    const float v = i < p.D ? row[h * p.D + i] * inv_q * to_f32(wq[h * p.D + i]) : 0.f;
    q_out[(size_t)t * p.ld_q + idx] = from_f32<T>(v);
  }
  if (!p.has_kv || cache_k == nullptr) return;
  ssk = block_sum(ssk, scratch);
  const float inv_k = 1.0f / sqrtf(ssk / (float)wk_n + p.eps);
  const int slot = p.slots[t];
  if (slot == -1) return;             // a row of padding: its keys and values go nowhere
  const int page = slot / p.page_size, off = slot - page * p.page_size;
  if (slot < 0 || page >= p.num_pages) {
    if (threadIdx.x == 0) lab_set_error(LAB_ERR_PAGE_RANGE);
    return;
  }
  for (int idx = threadIdx.x; idx < p.n_kv * p.HD; idx += kThreads) {
    const int g = idx / p.HD, i = idx - g * p.HD;
    const size_t dst = (((size_t)page * p.n_kv + g) * p.page_size + off) * p.HD + i;
    const float kv = i < p.D ? row[wq_n + g * p.D + i] * inv_k * to_f32(wk[g * p.D + i]) : 0.f;
    const float vv = i < p.V ? row[wq_n + wk_n + g * p.V + i] : 0.f;
    cache_k[dst] = from_f32<T>(kv);
    cache_v[dst] = from_f32<T>(vv);
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) head_gate_kernel(T* __restrict__ out, int ld_o, const T* __restrict__ attn,
                                                             int ld_a, const float* __restrict__ proj, int splits,
                                                             long long split_stride, int ld, int gate_at,
                                                             int per_head, long long tokens, int n_q, int V, int HD,
                                                             float mult) {
  pdl_trigger();
  pdl_wait();
  const int width = n_q * V;
  const long long n = tokens * width;
  for (long long e = (long long)blockIdx.x * kThreads + threadIdx.x; e < n; e += (long long)gridDim.x * kThreads) {
    const long long t = e / width;
    const int c = (int)(e - t * width), h = c / V, i = c - h * V;
    const float g = sum_splits(proj, splits, split_stride, (size_t)t * ld + gate_at + (per_head ? h : c));
    const float a = to_f32(attn[(size_t)t * ld_a + h * HD + i]);
    out[(size_t)t * ld_o + c] = from_f32<T>(a * mult / (1.0f + expf(-g)));
  }
}

int blocks_for(long long n) { return (int)((n + kThreads - 1) / kThreads < 148 * 8 ? (n + kThreads - 1) / kThreads : 148 * 8); }

}  // namespace

// proj: [splits][tokens, ld] floats (splits 1: the whole product); bias over the q, k and v columns or null.
LAB_EXPORT int lab_qk_norm_store(void* q_out, int ld_q, void* cache_k, void* cache_v, const float* proj, int splits,
                                 int ld, const void* bias, const void* wq, const void* wk, const int* slots, int tokens,
                                 int n_q, int n_kv, int D, int V, int HD, int page_size, int num_pages, int has_kv,
                                 float eps, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (HD < D || HD < V || n_q <= 0 || (has_kv && n_kv <= 0)) return (int)cudaErrorInvalidValue;
  QkNormParams p;
  p.proj = proj; p.splits = splits; p.split_stride = (long long)tokens * ld; p.ld = ld; p.slots = slots;
  p.n_q = n_q; p.n_kv = n_kv; p.D = D; p.V = V; p.HD = HD; p.page_size = page_size; p.num_pages = num_pages;
  p.has_kv = has_kv; p.ld_q = ld_q; p.eps = eps;
  const size_t smem = (size_t)(n_q * D + (has_kv ? n_kv * (D + V) : 0)) * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (dtype == LAB_F32) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(qk_norm_store_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    lab_launch(qk_norm_store_kernel<float>, dim3(tokens), dim3(kThreads), smem, stream, (float*)q_out, (float*)cache_k,
               (float*)cache_v, (const float*)bias, (const float*)wq, (const float*)wk, p);
  } else {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(qk_norm_store_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    lab_launch(qk_norm_store_kernel<__nv_bfloat16>, dim3(tokens), dim3(kThreads), smem, stream, (__nv_bfloat16*)q_out,
               (__nv_bfloat16*)cache_k, (__nv_bfloat16*)cache_v, (const __nv_bfloat16*)bias, (const __nv_bfloat16*)wq,
               (const __nv_bfloat16*)wk, p);
  }
  LAB_LAUNCH_CHECK();
}

// attn: [tokens, ld_a] of T with heads HD wide; the gate's pre-activations start at column gate_at of proj.
LAB_EXPORT int lab_head_gate(void* out, int ld_o, const void* attn, int ld_a, const float* proj, int splits, int ld,
                             int gate_at, int per_head, int tokens, int n_q, int V, int HD, float mult, int dtype,
                             cudaStream_t stream) {
  const long long n = (long long)tokens * n_q * V;
  if (n <= 0) return 0;
  const long long stride = (long long)tokens * ld;
  if (dtype == LAB_F32)
    lab_launch(head_gate_kernel<float>, dim3(blocks_for(n)), dim3(kThreads), 0, stream, (float*)out, ld_o,
               (const float*)attn, ld_a, proj, splits, stride, ld, gate_at, per_head, (long long)tokens, n_q, V, HD, mult);
  else
    lab_launch(head_gate_kernel<__nv_bfloat16>, dim3(blocks_for(n)), dim3(kThreads), 0, stream, (__nv_bfloat16*)out, ld_o,
               (const __nv_bfloat16*)attn, ld_a, proj, splits, stride, ld, gate_at, per_head, (long long)tokens, n_q, V,
               HD, mult);
  LAB_LAUNCH_CHECK();
}
