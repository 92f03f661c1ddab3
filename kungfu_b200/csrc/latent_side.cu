// Small row kernels of blocks with layer scales, a per-token side input and a latent key/value cache.
//
// kf_latent_append:      c = rms_norm(proj[t, c0 .. c0 + rank)) * w, written into the request's page at the token's
//                        position, once as the key row and once as the value row of a single key/value head of D >= rank
//                        elements (tails zero): attention in the latent space reads the same row as key and as value.
// kf_latent_rope_append: the same with a rotated key part that all heads share: the r columns after the latent are
//                        turned by the row's angles (pairs (2i, 2i + 1) when `interleaved`, else (i, i + r/2); cos and sin
//                        times `mag`) and filed behind c in the key row (the value row holds zeros there); the last r
//                        elements of every head of a 32-bit query matrix [T, H * (dq + r)] are turned in place likewise.
// kf_scale_add_rmsnorm:  x[t] += a[t] * s (s: one factor per column), 32-bit; optionally next = rms_norm(x[t]) * g in the
//                        same pass, and optionally a plain copy of the new x[t] in another element type.
// kf_side_gate:          out[t, j] = gelu_tanh(gate[t, j]) * table[token[t], col0 + j]: the gate of a per-token input whose
//                        second factor is looked up by token id.
// kf_repeat_rows:        out[t * parts + j] = in[t] for two integer arrays at once: the positions and requests of a step
//                        whose every row is presented to the attention kernels as `parts` rows of fewer heads.
#include "common.cuh"

__global__ void repeat_rows_kernel(const int* __restrict__ a, const int* __restrict__ b, int* __restrict__ out_a,
                                   int* __restrict__ out_b, int T, int parts) {
  kf_pdl_trigger();
  kf_pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * parts) return;
  out_a[i] = a[i / parts];
  out_b[i] = b[i / parts];
}

KF_API int kf_repeat_rows(const int* a, const int* b, int* out_a, int* out_b, int T, int parts, cudaStream_t stream) {
  if (T <= 0 || parts <= 0) return KF_OK;
  kf_launch(repeat_rows_kernel, dim3(kf_ceil_div((long)T * parts, 256)), dim3(256), 0, stream, a, b, out_a, out_b, T, parts);
  KF_CHECK_LAUNCH();
  return KF_OK;
}

template <typename TW, typename TC>
__global__ void latent_append_kernel(const float* __restrict__ proj, int ld, int c0, int rank, const TW* __restrict__ w, float eps,
                                     const int* __restrict__ positions, const int* __restrict__ row_req,
                                     const int* __restrict__ table, int table_width, int page_size, TC* __restrict__ pages, int D) {
  kf_pdl_trigger();
  kf_pdl_wait();
  __shared__ float red[33];
  const int t = blockIdx.x;
  const int req = row_req[t];
  if (req < 0) return;
  const float* src = proj + (size_t)t * ld + c0;
  float ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) ss = fmaf(src[i], src[i], ss);
  ss = kf_block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)rank + eps);
  const int pos = positions[t];
  const int page = table[(size_t)req * table_width + pos / page_size];
  if (page < 0) return;
  TC* kdst = pages + (((size_t)page * 2 + 0) * page_size + pos % page_size) * D;
  TC* vdst = pages + (((size_t)page * 2 + 1) * page_size + pos % page_size) * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float v = i < rank ? src[i] * inv * kf_load(w, i) : 0.f;
    kf_store(kdst, i, v);
    kf_store(vdst, i, v);
  }
}

KF_API int kf_latent_append(const float* proj, int ld, int c0, int rank, const void* w, int w_dtype, float eps,
                            const int* positions, const int* row_req, const int* table, int table_width, int page_size,
                            void* pages, int pages_dtype, int D, int T, cudaStream_t stream) {
  if (T <= 0) return KF_OK;
  if (rank < 1 || rank > D) return KF_ERR_SIZE;
#define KF_GO(TW, TC)                                                                                                        \
  kf_launch(latent_append_kernel<TW, TC>, dim3(T), dim3(128), 0, stream, proj, ld, c0, rank, (const TW*)w, eps, positions, \
            row_req, table, table_width, page_size, (TC*)pages, D)
  if (w_dtype == KF_F32 && pages_dtype == KF_F32) KF_GO(float, float);
  else if (w_dtype == KF_BF16 && pages_dtype == KF_BF16) KF_GO(__nv_bfloat16, __nv_bfloat16);
  else if (w_dtype == KF_BF16 && pages_dtype == KF_F32) KF_GO(__nv_bfloat16, float);
  else if (w_dtype == KF_F32 && pages_dtype == KF_BF16) KF_GO(float, __nv_bfloat16);
  else return KF_ERR_DTYPE;
#undef KF_GO
  KF_CHECK_LAUNCH();
  return KF_OK;
}

template <typename TW, typename TC>
__global__ void __launch_bounds__(128)
latent_rope_append_kernel(const float* __restrict__ proj, int ld, int c0, int rank, int r, const TW* __restrict__ w, float eps,
                          const float* __restrict__ cos_t, const float* __restrict__ sin_t, int interleaved, float mag,
                          float* __restrict__ q, int ldq, int q0, int H, int dq, const int* __restrict__ positions,
                          const int* __restrict__ row_req, const int* __restrict__ table, int table_width, int page_size,
                          TC* __restrict__ pages, int D, int write_kv) {
  kf_pdl_trigger();
  kf_pdl_wait();
  __shared__ float red[33];
  const int t = blockIdx.x;
  const int req = row_req[t];
  if (req < 0) return;
  const int half = r >> 1;
  const float* c = cos_t + (size_t)t * half;
  const float* s = sin_t + (size_t)t * half;
  // the queries' rotated parts, in place: one thread per pair
  for (int i = threadIdx.x; i < H * half; i += blockDim.x) {
    const int h = i / half, pr = i - h * half;
    float* x = q + (size_t)t * ldq + q0 + (size_t)h * (dq + r) + dq;
    const int a = interleaved ? 2 * pr : pr, b = interleaved ? 2 * pr + 1 : pr + half;
    const float u = x[a], v = x[b], cs = c[pr] * mag, sn = s[pr] * mag;
    x[a] = u * cs - v * sn;
    x[b] = v * cs + u * sn;
  }
  if (!write_kv) return;
  const float* src = proj + (size_t)t * ld + c0;
  float ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) ss = fmaf(src[i], src[i], ss);
  ss = kf_block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)rank + eps);
  const int pos = positions[t];
  const int page = table[(size_t)req * table_width + pos / page_size];
  if (page < 0) return;
  TC* kdst = pages + (((size_t)page * 2 + 0) * page_size + pos % page_size) * D;
  TC* vdst = pages + (((size_t)page * 2 + 1) * page_size + pos % page_size) * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float kv = 0.f, vv = 0.f;
    if (i < rank) kv = vv = src[i] * inv * kf_load(w, i);
    else if (i < rank + r) {
      const int e = i - rank;
      int pr, partner;
      bool first;
      if (interleaved) { pr = e >> 1; first = !(e & 1); partner = e ^ 1; }
      else { first = e < half; pr = first ? e : e - half; partner = first ? e + half : e - half; }
      const float x = src[rank + e], o = src[rank + partner], cs = c[pr] * mag, sn = s[pr] * mag;
      kv = first ? x * cs - o * sn : x * cs + o * sn;
    }
    kf_store(kdst, i, kv);
    kf_store(vdst, i, vv);
  }
}

KF_API int kf_latent_rope_append(const float* proj, int ld, int c0, int rank, int r, const void* w, int w_dtype, float eps,
                                 const float* cos_t, const float* sin_t, int interleaved, float mag, float* q, int ldq, int q0,
                                 int H, int dq, const int* positions, const int* row_req, const int* table, int table_width,
                                 int page_size, void* pages, int pages_dtype, int D, int write_kv, int T, cudaStream_t stream) {
  if (T <= 0) return KF_OK;
  if (rank < 1 || r < 0 || (r & 1) || rank + r > D || (r > 0 && (!cos_t || !sin_t))) return KF_ERR_SIZE;
#define KF_GO(TW, TC)                                                                                                       \
  kf_launch(latent_rope_append_kernel<TW, TC>, dim3(T), dim3(128), 0, stream, proj, ld, c0, rank, r, (const TW*)w, eps, cos_t, \
            sin_t, interleaved, mag, q, ldq, q0, H, dq, positions, row_req, table, table_width, page_size, (TC*)pages, D,  \
            write_kv)
  if (w_dtype == KF_F32 && pages_dtype == KF_F32) KF_GO(float, float);
  else if (w_dtype == KF_BF16 && pages_dtype == KF_BF16) KF_GO(__nv_bfloat16, __nv_bfloat16);
  else if (w_dtype == KF_BF16 && pages_dtype == KF_F32) KF_GO(__nv_bfloat16, float);
  else if (w_dtype == KF_F32 && pages_dtype == KF_BF16) KF_GO(float, __nv_bfloat16);
  else return KF_ERR_DTYPE;
#undef KF_GO
  KF_CHECK_LAUNCH();
  return KF_OK;
}

template <typename TS, typename TW, typename TO, typename TC>
__global__ void scale_add_rmsnorm_kernel(const float* __restrict__ a, const TS* __restrict__ s, float* __restrict__ x,
                                         const TW* __restrict__ w, float eps, int plus_one, TO* __restrict__ out,
                                         TC* __restrict__ copy, int H) {
  kf_pdl_trigger();
  kf_pdl_wait();
  __shared__ float red[33];
  const size_t base = (size_t)blockIdx.x * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = fmaf(a[base + i], kf_load(s, i), x[base + i]);
    x[base + i] = v;
    if (copy) kf_store(copy, base + i, v);
    ss = fmaf(v, v, ss);
  }
  if (!out) return;
  ss = kf_block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float g = kf_load(w, i) + (plus_one ? 1.f : 0.f);
    kf_store(out, base + i, x[base + i] * inv * g);
  }
}

// s, w share one element type (the model's); out and copy share one (the step's activation type).
KF_API int kf_scale_add_rmsnorm(const float* a, const void* s, int s_dtype, float* x, const void* w, float eps, int plus_one,
                                void* out, void* copy, int out_dtype, int T, int H, cudaStream_t stream) {
  if (T <= 0) return KF_OK;
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
#define KF_GO(TS, TO)                                                                                                     \
  kf_launch(scale_add_rmsnorm_kernel<TS, TS, TO, TO>, dim3(T), dim3(threads), 0, stream, a, (const TS*)s, x, (const TS*)w, \
            eps, plus_one, (TO*)out, (TO*)copy, H)
  if (s_dtype == KF_F32 && out_dtype == KF_F32) KF_GO(float, float);
  else if (s_dtype == KF_BF16 && out_dtype == KF_BF16) KF_GO(__nv_bfloat16, __nv_bfloat16);
  else if (s_dtype == KF_BF16 && out_dtype == KF_F32) KF_GO(__nv_bfloat16, float);
  else if (s_dtype == KF_F32 && out_dtype == KF_BF16) KF_GO(float, __nv_bfloat16);
  else return KF_ERR_DTYPE;
#undef KF_GO
  KF_CHECK_LAUNCH();
  return KF_OK;
}

template <typename TE, typename TO>
__global__ void side_gate_kernel(const float* __restrict__ gate, const int* __restrict__ tokens, const TE* __restrict__ table,
                                 int table_ld, int col0, TO* __restrict__ out, int T, int dim) {
  kf_pdl_trigger();
  kf_pdl_wait();
  const long n = (long)T * dim;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (long)gridDim.x * blockDim.x) {
    const long t = idx / dim, j = idx - t * dim;
    const float e = kf_load(table, (size_t)tokens[t] * table_ld + col0 + j);
    kf_store(out, idx, kf_act(gate[idx], KF_ACT_GELU_TANH) * e);
  }
}

KF_API int kf_side_gate(const float* gate, const int* tokens, const void* table, int table_dtype, int table_ld, int col0,
                        void* out, int out_dtype, int T, int dim, cudaStream_t stream) {
  if (T <= 0 || dim <= 0) return KF_OK;
  const long n = (long)T * dim;
  const int blocks = (int)((n + 255) / 256 > 4096 ? 4096 : (n + 255) / 256);
#define KF_GO(TE, TO) \
  kf_launch(side_gate_kernel<TE, TO>, dim3(blocks), dim3(256), 0, stream, gate, tokens, (const TE*)table, table_ld, col0, (TO*)out, T, dim)
  if (table_dtype == KF_F32 && out_dtype == KF_F32) KF_GO(float, float);
  else if (table_dtype == KF_BF16 && out_dtype == KF_BF16) KF_GO(__nv_bfloat16, __nv_bfloat16);
  else if (table_dtype == KF_BF16 && out_dtype == KF_F32) KF_GO(__nv_bfloat16, float);
  else if (table_dtype == KF_F32 && out_dtype == KF_BF16) KF_GO(float, __nv_bfloat16);
  else return KF_ERR_DTYPE;
#undef KF_GO
  KF_CHECK_LAUNCH();
  return KF_OK;
}
