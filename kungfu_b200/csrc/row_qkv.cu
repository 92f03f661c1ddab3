// From a 32-bit stacked projection to the attention's operands, for mixers that norm q and k over the WHOLE projection
// (all heads of a row at once) instead of head by head.
//
// kf_rownorm_rope_append, one block per row of the step:
//   q = in[t, col0 ..] + bias_q,  k = ... + bias_k,  v = ... + bias_v                    (bias optional)
//   q <- q / sqrt(mean over all nh * dk elements of q^2 + eps) * wq[i]   (wq: nh * dk weights; null: no norm), k likewise
//   the first `rot` elements of every head of q and k are turned by the row's angles, pairs (2i, 2i + 1) when
//   `interleaved`, else (i, i + rot/2); cos and sin are multiplied by `mag`
//   value mixing: vmode 1 writes the biased v of the row to v_shared [T, nkv * dv] (32-bit); vmode 2 replaces v by
//   (1 - lambda) v + lambda v_shared[t] (lambda: one number on the device); what was mixed is what is filed
//   q goes to q_out [T, nh * D], k and v to the token's place in the request's pages; heads use D elements, tails zero.
// kf_cols_rmsnorm: out[t, i] = in[t, c0 + i] / sqrt(mean_i(in[t, c0 + i]^2) + eps) * w[i] for a column range of a 32-bit
//   matrix (the normed latent a second projection reads).
// Everything is computed in 32-bit; only the stores round.
#include "common.cuh"

template <typename TW, typename TQ, typename TKV>
__global__ void __launch_bounds__(256)
rownorm_rope_append_kernel(const float* __restrict__ in, int ld, int col0, const TW* __restrict__ bias,
                           const TW* __restrict__ wq, const TW* __restrict__ wk, float eps, const float* __restrict__ cos_t,
                           const float* __restrict__ sin_t, int rot, int interleaved, float mag, int nh, int nkv, int dk,
                           int dv, int D, const TW* __restrict__ lambda, float* __restrict__ v_shared, int vmode,
                           const int* __restrict__ positions, const int* __restrict__ row_req,
                           const int* __restrict__ block_table, int table_stride, int page_size, TKV* __restrict__ pages,
                           TQ* __restrict__ q_out, int write_kv, int T) {
  kf_pdl_trigger();
  kf_pdl_wait();
  extern __shared__ float row[];                            // q (nh * dk) then k (nkv * dk), biased
  __shared__ float red[33];
  const int t = blockIdx.x;
  const int req = row_req[t];
  const int nq = nh * dk, nk = nkv * dk, nv = nkv * dv;
  if (req < 0) {                                            // padding row: zero queries, nothing filed
    for (int i = threadIdx.x; i < nh * D; i += blockDim.x) kf_store(q_out, (size_t)t * nh * D + i, 0.f);
    return;
  }
  const float* src = in + (size_t)t * ld + col0;
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < nq + nk; i += blockDim.x) {
    const float x = src[i] + (bias ? kf_load(bias, i) : 0.f);
    row[i] = x;
    if (i < nq) sq = fmaf(x, x, sq); else sk = fmaf(x, x, sk);
  }
  sq = kf_block_sum(sq, red);
  sk = kf_block_sum(sk, red);
  const float inv_q = wq ? 1.f / sqrtf(sq / (float)nq + eps) : 1.f;
  const float inv_k = wk ? 1.f / sqrtf(sk / (float)nk + eps) : 1.f;
  const int half = rot >> 1;
  const float* c = cos_t + (size_t)t * half;
  const float* s = sin_t + (size_t)t * half;
  const int pos = positions[t];
  const int page = block_table[(size_t)req * table_stride + pos / page_size];
  const int in_page = pos % page_size;
  const bool file = write_kv && page >= 0;
  const int n_heads_qk = nh + (file ? nkv : 0);
  for (int i = threadIdx.x; i < n_heads_qk * D; i += blockDim.x) {
    const int hs = i / D, e = i - hs * D;
    const bool is_q = hs < nh;
    const int head = is_q ? hs : hs - nh;
    float y = 0.f;
    if (e < dk) {
      const int base = (is_q ? 0 : nq) + head * dk;
      const TW* w = is_q ? wq : wk;
      const float inv = is_q ? inv_q : inv_k;
      const int wbase = head * dk;
      auto normed = [&](int j) { return row[base + j] * inv * (w ? kf_load(w, wbase + j) : 1.f); };
      y = normed(e);
      if (e < rot) {
        int pair, partner;
        bool first;
        if (interleaved) { pair = e >> 1; first = !(e & 1); partner = e ^ 1; }
        else { first = e < half; pair = first ? e : e - half; partner = first ? e + half : e - half; }
        const float cs = c[pair] * mag, sn = s[pair] * mag, o = normed(partner);
        y = first ? y * cs - o * sn : y * cs + o * sn;
      }
    }
    if (is_q) kf_store(q_out, ((size_t)t * nh + head) * D + e, y);
    else kf_store(pages, ((((size_t)page * 2 + 0) * nkv + head) * page_size + in_page) * D + e, y);
  }
  if (!write_kv) return;
  const float lam = (vmode == 2 && lambda) ? kf_load(lambda, 0) : 0.f;
  for (int i = threadIdx.x; i < nkv * D; i += blockDim.x) {
    const int head = i / D, e = i - head * D;
    float y = 0.f;
    if (e < dv) {
      const int j = head * dv + e;
      y = src[nq + nk + j] + (bias ? kf_load(bias, nq + nk + j) : 0.f);
      if (vmode == 1) v_shared[(size_t)t * nv + j] = y;
      else if (vmode == 2) y = (1.f - lam) * y + lam * v_shared[(size_t)t * nv + j];
    }
    if (page >= 0) kf_store(pages, ((((size_t)page * 2 + 1) * nkv + head) * page_size + in_page) * D + e, y);
  }
}

KF_API int kf_rownorm_rope_append(const float* in, int ld, int col0, const void* bias, const void* wq, const void* wk,
                                  int w_dtype, float eps, const float* cos_t, const float* sin_t, int rot, int interleaved,
                                  float mag, int nh, int nkv, int dk, int dv, int D, const void* lambda, float* v_shared,
                                  int vmode, const int* positions, const int* row_req, const int* block_table,
                                  int table_stride, int page_size, void* pages, int kv_dtype, void* q_out, int q_dtype,
                                  int write_kv, int T, cudaStream_t stream) {
  if (T <= 0) return KF_OK;
  if (dk > D || dv > D || dk < 1 || dv < 1 || rot > dk || (rot & 1) || nkv < 1 || nh % nkv) return KF_ERR_SIZE;
  if (rot > 0 && (!cos_t || !sin_t)) return KF_ERR_SIZE;
  if (vmode != 0 && !v_shared) return KF_ERR_SIZE;
  const size_t smem = (size_t)(nh + nkv) * dk * sizeof(float);
  if (smem > 200 * 1024) return KF_ERR_SIZE;
#define KF_GO(TW, TQ, TKV)                                                                                              \
  do {                                                                                                                  \
    if (smem > 48 * 1024)                                                                                               \
      cudaFuncSetAttribute(rownorm_rope_append_kernel<TW, TQ, TKV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    kf_launch(rownorm_rope_append_kernel<TW, TQ, TKV>, dim3(T), dim3(256), smem, stream, in, ld, col0, (const TW*)bias,  \
              (const TW*)wq, (const TW*)wk, eps, cos_t, sin_t, rot, interleaved, mag, nh, nkv, dk, dv, D,              \
              (const TW*)lambda, v_shared, vmode, positions, row_req, block_table, table_stride, page_size,            \
              (TKV*)pages, (TQ*)q_out, write_kv, T);                                                                    \
  } while (0)
  if (w_dtype == KF_F32 && q_dtype == KF_F32 && kv_dtype == KF_F32) KF_GO(float, float, float);
  else if (w_dtype == KF_BF16 && q_dtype == KF_BF16 && kv_dtype == KF_BF16) KF_GO(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
  else if (w_dtype == KF_BF16 && q_dtype == KF_F32 && kv_dtype == KF_F32) KF_GO(__nv_bfloat16, float, float);
  else if (w_dtype == KF_F32 && q_dtype == KF_BF16 && kv_dtype == KF_BF16) KF_GO(float, __nv_bfloat16, __nv_bfloat16);
  else return KF_ERR_DTYPE;
#undef KF_GO
  KF_CHECK_LAUNCH();
  return KF_OK;
}

template <typename TW, typename TO>
__global__ void __launch_bounds__(128) cols_rmsnorm_kernel(const float* __restrict__ in, int ld, int c0, int n,
                                                           const TW* __restrict__ w, float eps, TO* __restrict__ out) {
  kf_pdl_trigger();
  kf_pdl_wait();
  __shared__ float red[33];
  const int t = blockIdx.x;
  const float* src = in + (size_t)t * ld + c0;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) ss = fmaf(src[i], src[i], ss);
  ss = kf_block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x) kf_store(out, (size_t)t * n + i, src[i] * inv * kf_load(w, i));
}

KF_API int kf_cols_rmsnorm(const float* in, int ld, int c0, int n, const void* w, int w_dtype, float eps, void* out,
                           int out_dtype, int T, cudaStream_t stream) {
  if (T <= 0) return KF_OK;
  if (n < 1 || c0 < 0 || c0 + n > ld) return KF_ERR_SIZE;
#define KF_GO(TW, TO) kf_launch(cols_rmsnorm_kernel<TW, TO>, dim3(T), dim3(128), 0, stream, in, ld, c0, n, (const TW*)w, eps, (TO*)out)
  if (w_dtype == KF_F32 && out_dtype == KF_F32) KF_GO(float, float);
  else if (w_dtype == KF_BF16 && out_dtype == KF_BF16) KF_GO(__nv_bfloat16, __nv_bfloat16);
  else if (w_dtype == KF_BF16 && out_dtype == KF_F32) KF_GO(__nv_bfloat16, float);
  else if (w_dtype == KF_F32 && out_dtype == KF_BF16) KF_GO(float, __nv_bfloat16);
  else return KF_ERR_DTYPE;
#undef KF_GO
  KF_CHECK_LAUNCH();
  return KF_OK;
}
