// What stands between the q|k|v projection and the attention kernels, for mixers that do more there than rotate:
// one warp per (row, head) takes a head of q, k or v through
//   1. an optional bias and short causal convolution over time (short_conv.cuh; the state is read here and moved on
//      afterwards by kf_short_conv_commit),
//   2. for q and k an optional RMS norm over the head, x / sqrt(mean(x^2) + eps) * w, one weight vector shared by all heads,
//   3. for q and k the rotation of the first `rot` elements by the step's cos/sin table, pairs (2i, 2i+1) when
//      `interleaved`, else (i, i + rot/2),
// and stores q as a row of the attention's query matrix and k, v at the token's place in the request's pages.
// Keys and values may have different sizes dk and dv; queries and pages use D >= max(dk, dv) elements per head and the
// tail is zero (a zero tail changes neither q.k nor the first dv elements of the weighted sum of values).
// Input layout per row: [ nh*dk | nkv*dk | nkv*dv ] starting at column col0 of a 32-bit matrix with ld columns.
// Page layout: pages[page][0 = key | 1 = value][kv head][slot in page][D].
// Everything is computed in 32-bit; only the stores round.
#include "short_conv.cuh"

__device__ __forceinline__ void kf_store_vec4(float* o, size_t i, float4 v) { *reinterpret_cast<float4*>(o + i) = v; }
__device__ __forceinline__ void kf_store_vec4(__nv_bfloat16* o, size_t i, float4 v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(o + i) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}

// Four neighbouring elements p[i .. i+3] (i a multiple of four, the base 16-byte aligned) in one load.
__device__ __forceinline__ float4 kf_load4(const float* p, size_t i) { return *reinterpret_cast<const float4*>(p + i); }
__device__ __forceinline__ float4 kf_load4(const __nv_bfloat16* p, size_t i) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p + i);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}

constexpr int QP_MAX_D = 256;
constexpr int QP_WARPS = 4;

template <typename TW, typename TQ, typename TKV>
__global__ void __launch_bounds__(QP_WARPS * 32)
qkv_prepare_kernel(KfConvIn cv, const TW* __restrict__ conv_w, const TW* __restrict__ q_norm, const TW* __restrict__ k_norm,
                   float eps, const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot, int interleaved,
                   int nh, int nkv, int dk, int dv, int D, const int* __restrict__ positions,
                   const int* __restrict__ row_req, const int* __restrict__ req_row_start,
                   const int* __restrict__ req_state_slot, const int* __restrict__ block_table, int table_stride,
                   int page_size, TKV* __restrict__ pages, TQ* __restrict__ q_out, int write_kv, int T) {
  kf_pdl_trigger();
  kf_pdl_wait();
  __shared__ float hs[QP_WARPS][QP_MAX_D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slots = nh + 2 * nkv;
  const long item = (long)blockIdx.x * QP_WARPS + warp;
  if (item >= (long)T * slots) return;                      // whole warps leave; only __syncwarp below
  const int t = (int)(item / slots), hslot = (int)(item - (long)t * slots);
  const int req = row_req[t];
  const int kind = hslot < nh ? 0 : (hslot < nh + nkv ? 1 : 2);            // query, key, value
  const int head = kind == 0 ? hslot : (kind == 1 ? hslot - nh : hslot - nh - nkv);
  if (req < 0) {                                            // padding row: a zero query, nothing filed
    if (kind == 0)
      for (int i = lane; i < D; i += 32) kf_store(q_out, ((size_t)t * nh + head) * D + i, 0.f);
    return;
  }
  if (kind != 0 && !write_kv) return;
  const int d = kind == 2 ? dv : dk;
  const int chan0 = kind == 0 ? head * dk : (kind == 1 ? nh * dk + head * dk : (nh + nkv) * dk + head * dv);
  const int row0 = req_row_start[req], slot = req_state_slot[req];
  float* x = hs[warp];
  float ss = 0.f;
  for (int i = lane; i < d; i += 32) {
    float v;
    if (conv_w) v = kf_conv_value<TW>(cv, conv_w, row0, slot, t - row0, chan0 + i);
    else v = kf_conv_input<TW>(cv, t, 0, 0, chan0 + i);     // no convolution: the row's own (biased) value
    x[i] = v;
    ss = fmaf(v, v, ss);
  }
  const TW* nw = kind == 0 ? q_norm : (kind == 1 ? k_norm : nullptr);
  if (nw) {
    ss = kf_warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)d + eps);
    for (int i = lane; i < d; i += 32) x[i] = x[i] * inv * kf_load(nw, i);
  }
  __syncwarp();
  // destination of this head
  TQ* qo = nullptr;
  TKV* po = nullptr;
  if (kind == 0) {
    qo = q_out + ((size_t)t * nh + head) * D;
  } else {
    const int pos = positions[t];
    const int page = block_table[(size_t)req * table_stride + pos / page_size];
    if (page < 0) return;                                   // never for a reserved position; guards the store
    po = pages + ((((size_t)page * 2 + (kind - 1)) * nkv + head) * page_size + (pos % page_size)) * D;
  }
  const int half = rot >> 1;
  const float* c = cos_t + (size_t)t * half;
  const float* s = sin_t + (size_t)t * half;
  for (int i = lane; i < D; i += 32) {
    float v = 0.f;
    if (i < d) {
      v = x[i];
      if (kind != 2 && i < rot) {
        if (interleaved) {
          const int pr = i >> 1;
          v = (i & 1) ? fmaf(x[i], c[pr], x[i - 1] * s[pr]) : fmaf(x[i], c[pr], -x[i + 1] * s[pr]);
        } else {
          v = i < half ? fmaf(x[i], c[i], -x[i + half] * s[i]) : fmaf(x[i], c[i - half], x[i - half] * s[i - half]);
        }
      }
    }
    if (kind == 0) kf_store(qo, i, v);
    else kf_store(po, i, v);
  }
}

// The same with four neighbouring elements of a head per lane (16-byte loads, 8- or 16-byte stores), for head sizes,
// rotated sizes and offsets that are multiples of four and interleaved pairs (a pair then lies within a lane's four
// elements, so nothing is exchanged between lanes but the sum of squares).  A block owns one row and its warps take the
// row's heads in turn, so the row's look-ups happen once.  `commit_state`: as in the short convolution, for steps
// without a request of more than one row the lanes also move the convolution's tail on.
template <typename TW, typename TQ, typename TKV>
__global__ void __launch_bounds__(QP_WARPS * 32)
qkv_prepare_vec_kernel(KfConvIn cv, const TW* __restrict__ conv_w, const TW* __restrict__ q_norm, const TW* __restrict__ k_norm,
                       float eps, const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot,
                       int nh, int nkv, int dk, int dv, int D, const int* __restrict__ positions,
                       const int* __restrict__ row_req, const int* __restrict__ req_row_start,
                       const int* __restrict__ req_state_slot, const int* __restrict__ block_table, int table_stride,
                       int page_size, TKV* __restrict__ pages, TQ* __restrict__ q_out, int write_kv,
                       float* __restrict__ commit_state) {
  kf_pdl_trigger();
  kf_pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int req = row_req[t];
  const int slots = nh + 2 * nkv;
  const int stride = QP_WARPS * gridDim.y;                 // gridDim.y blocks share a row's heads (few rows: more blocks)
  if (req < 0) {                                            // padding row: a zero query, nothing filed
    for (int i = (blockIdx.y * QP_WARPS * 32 + threadIdx.x) * 4; i < nh * D; i += stride * 128)
      kf_store_vec4(q_out, (size_t)t * nh * D + i, make_float4(0.f, 0.f, 0.f, 0.f));
    return;
  }
  const int row0 = req_row_start[req], slot = req_state_slot[req], li = t - row0;
  const int pos = positions[t];
  const int page = block_table[(size_t)req * table_stride + pos / page_size];
  const int half = rot >> 1;
  const float* c = cos_t + (size_t)t * half;
  const float* sn = sin_t + (size_t)t * half;
  for (int hslot = blockIdx.y * QP_WARPS + warp; hslot < slots; hslot += stride) {
    const int kind = hslot < nh ? 0 : (hslot < nh + nkv ? 1 : 2);
    const int head = kind == 0 ? hslot : (kind == 1 ? hslot - nh : hslot - nh - nkv);
    if (kind != 0 && (!write_kv || page < 0) && !commit_state) continue;
    const int d = kind == 2 ? dv : dk;
    const int chan0 = kind == 0 ? head * dk : (kind == 1 ? nh * dk + head * dk : (nh + nkv) * dk + head * dv);
    float4 x[2];                                            // elements 4 lane + 128 r .. + 3
    float ss = 0.f;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int i = 4 * lane + 128 * r;
      x[r] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i < d) {
        const int ch = chan0 + i;
        const float4 bi = cv.in_bias ? kf_load4((const TW*)cv.in_bias, ch) : make_float4(0.f, 0.f, 0.f, 0.f);
        // the filter taps of the lane's four channels: with four taps one load per channel
        float4 w0, w1, w2, w3;                              // w_c = taps 0..3 of channel ch + c
        const bool four = conv_w && cv.taps == 4;
        if (four) {
          w0 = kf_load4(conv_w, (size_t)ch * 4); w1 = kf_load4(conv_w, (size_t)ch * 4 + 4);
          w2 = kf_load4(conv_w, (size_t)ch * 4 + 8); w3 = kf_load4(conv_w, (size_t)ch * 4 + 12);
        }
        for (int j = 0; j < cv.taps; ++j) {
          const int idx = li - (cv.taps - 1 - j);
          float4 u;
          if (idx >= 0) {
            u = *reinterpret_cast<const float4*>(cv.in + (size_t)(row0 + idx) * cv.ld + cv.col0 + ch);
            u.x += bi.x; u.y += bi.y; u.z += bi.z; u.w += bi.w;
          } else {
            u = *reinterpret_cast<const float4*>(cv.state + ((size_t)slot * (cv.taps - 1) + (cv.taps - 1 + idx)) * cv.C + ch);
          }
          if (four) {
            const float t0 = j == 0 ? w0.x : j == 1 ? w0.y : j == 2 ? w0.z : w0.w, t1 = j == 0 ? w1.x : j == 1 ? w1.y : j == 2 ? w1.z : w1.w;
            const float t2 = j == 0 ? w2.x : j == 1 ? w2.y : j == 2 ? w2.z : w2.w, t3 = j == 0 ? w3.x : j == 1 ? w3.y : j == 2 ? w3.z : w3.w;
            x[r].x = fmaf(t0, u.x, x[r].x); x[r].y = fmaf(t1, u.y, x[r].y);
            x[r].z = fmaf(t2, u.z, x[r].z); x[r].w = fmaf(t3, u.w, x[r].w);
          } else if (conv_w) {
            x[r].x = fmaf(kf_load(conv_w, (size_t)ch * cv.taps + j), u.x, x[r].x);
            x[r].y = fmaf(kf_load(conv_w, (size_t)(ch + 1) * cv.taps + j), u.y, x[r].y);
            x[r].z = fmaf(kf_load(conv_w, (size_t)(ch + 2) * cv.taps + j), u.z, x[r].z);
            x[r].w = fmaf(kf_load(conv_w, (size_t)(ch + 3) * cv.taps + j), u.w, x[r].w);
          } else {
            x[r] = u;
          }
          if (commit_state && j >= 1)
            *reinterpret_cast<float4*>(commit_state + ((size_t)slot * (cv.taps - 1) + (j - 1)) * cv.C + ch) = u;
        }
        ss += x[r].x * x[r].x + x[r].y * x[r].y + x[r].z * x[r].z + x[r].w * x[r].w;
      }
    }
    if (kind != 0 && (!write_kv || page < 0)) continue;     // only the tail had to move on
    const TW* nw = kind == 0 ? q_norm : (kind == 1 ? k_norm : nullptr);
    if (nw) {
      ss = kf_warp_sum(ss);
      const float inv = 1.f / sqrtf(ss / (float)d + eps);
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int i = 4 * lane + 128 * r;
        if (i < d) {
          const float4 g = kf_load4(nw, i);
          x[r].x *= inv * g.x; x[r].y *= inv * g.y; x[r].z *= inv * g.z; x[r].w *= inv * g.w;
        }
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int i = 4 * lane + 128 * r;
      if (i >= D) continue;
      float4 v = x[r];                                       // zero beyond d
      if (kind != 2 && i < rot) {
        const float2 cc = *reinterpret_cast<const float2*>(c + (i >> 1)), sv = *reinterpret_cast<const float2*>(sn + (i >> 1));
        v = make_float4(fmaf(x[r].x, cc.x, -x[r].y * sv.x), fmaf(x[r].y, cc.x, x[r].x * sv.x),
                        fmaf(x[r].z, cc.y, -x[r].w * sv.y), fmaf(x[r].w, cc.y, x[r].z * sv.y));
      }
      if (kind == 0) kf_store_vec4(q_out, ((size_t)t * nh + head) * D + i, v);
      else kf_store_vec4(pages, ((((size_t)page * 2 + (kind - 1)) * nkv + head) * page_size + (pos % page_size)) * D + i, v);
    }
  }
}

// commit_inline: the step has no request with more than one row; the convolution's state is then moved on here and
// kf_short_conv_commit must not run for this step.
KF_API int kf_qkv_prepare(const float* in, int ld, int col0, const void* in_bias, const void* conv_w, int taps,
                          float* conv_state, const void* q_norm, const void* k_norm, int w_dtype, float eps,
                          const float* cos_t, const float* sin_t, int rot, int interleaved, int nh, int nkv, int dk, int dv,
                          int D, const int* positions, const int* row_req, const int* req_row_start,
                          const int* req_state_slot, const int* block_table, int table_stride, int page_size,
                          void* pages, int kv_dtype, void* q_out, int q_dtype, int write_kv, int T, int commit_inline,
                          cudaStream_t stream) {
  if (T <= 0) return KF_OK;
  if (D > QP_MAX_D || dk > D || dv > D || dk < 1 || dv < 1 || rot > dk || (rot & 1) || taps > KF_MAX_TAPS) return KF_ERR_SIZE;
  if (rot > 0 && (!cos_t || !sin_t)) return KF_ERR_SIZE;
  if (!conv_w) taps = 1;
  KfConvIn cv{in, ld, col0, in_bias, conv_state, nh * dk + nkv * dk + nkv * dv, taps};
  const bool vec = dk % 4 == 0 && dv % 4 == 0 && D % 4 == 0 && rot % 4 == 0 && (interleaved || rot == 0) && ld % 4 == 0 &&
                   col0 % 4 == 0 && (((uintptr_t)in | (uintptr_t)conv_state | (uintptr_t)q_out | (uintptr_t)pages) & 15) == 0 &&
                   (((uintptr_t)in_bias | (uintptr_t)conv_w | (uintptr_t)q_norm | (uintptr_t)k_norm) & 15) == 0 &&
                   (((uintptr_t)cos_t | (uintptr_t)sin_t) & 7) == 0;
  const bool commit = commit_inline && conv_w && taps > 1;
  if (commit && !vec) return KF_ERR_ALIGN;                  // the caller asks `kf_qkv_prepare_commits_inline` first
#define KF_GOV(TW, TQ, TKV)                                                                                             \
  kf_launch(qkv_prepare_vec_kernel<TW, TQ, TKV>, dim3(T, T >= 512 ? 1 : kf_ceil_div(nh + 2 * nkv, QP_WARPS)),              \
            dim3(QP_WARPS * 32), 0, stream, cv, (const TW*)conv_w,                                                       \
            (const TW*)q_norm, (const TW*)k_norm, eps, cos_t, sin_t, rot, nh, nkv, dk, dv, D, positions, row_req,          \
            req_row_start, req_state_slot, block_table, table_stride, page_size, (TKV*)pages, (TQ*)q_out, write_kv,      \
            commit ? conv_state : (float*)nullptr)
  if (vec) {
    if (w_dtype == KF_F32 && q_dtype == KF_F32 && kv_dtype == KF_F32) KF_GOV(float, float, float);
    else if (w_dtype == KF_BF16 && q_dtype == KF_BF16 && kv_dtype == KF_BF16) KF_GOV(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
    else return KF_ERR_DTYPE;
    KF_CHECK_LAUNCH();
    return KF_OK;
  }
#undef KF_GOV
  const long n_work = (long)T * (nh + 2 * nkv);
  const dim3 grid((unsigned)((n_work + QP_WARPS - 1) / QP_WARPS));
#define KF_GO(TW, TQ, TKV)                                                                                              \
  kf_launch(qkv_prepare_kernel<TW, TQ, TKV>, grid, dim3(QP_WARPS * 32), 0, stream, cv, (const TW*)conv_w,                \
            (const TW*)q_norm, (const TW*)k_norm, eps, cos_t, sin_t, rot, interleaved, nh, nkv, dk, dv, D, positions,     \
            row_req, req_row_start, req_state_slot, block_table, table_stride, page_size, (TKV*)pages, (TQ*)q_out,      \
            write_kv, T)
  if (w_dtype == KF_F32 && q_dtype == KF_F32 && kv_dtype == KF_F32) KF_GO(float, float, float);
  else if (w_dtype == KF_BF16 && q_dtype == KF_BF16 && kv_dtype == KF_BF16) KF_GO(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
  else return KF_ERR_DTYPE;
#undef KF_GO
  KF_CHECK_LAUNCH();
  return KF_OK;
}

// Whether kf_qkv_prepare with these sizes runs the kernel that can move the convolution's tail on itself.
KF_API int kf_qkv_prepare_commits_inline(int ld, int col0, int rot, int interleaved, int dk, int dv, int D) {
  return dk % 4 == 0 && dv % 4 == 0 && D % 4 == 0 && rot % 4 == 0 && (interleaved || rot == 0) && ld % 4 == 0 && col0 % 4 == 0;
}

// The per-head output gate and the packing of the attention's result: out[t][h*dv + i] = o[t][h*D + i] * sigmoid(g[t][h]),
// g read from column gcol0 + h of a 32-bit matrix with ld columns (null: no gate, only the packing).
template <typename TQ>
__global__ void head_gate_kernel(const TQ* __restrict__ o, const float* __restrict__ g, int ld, int gcol0, int nh, int dv,
                                 int D, TQ* __restrict__ out, const int* __restrict__ row_req, int ldo, int ocol0, float scale) {
  kf_pdl_trigger();
  kf_pdl_wait();
  const int t = blockIdx.x;
  const bool pad = row_req[t] < 0;
  for (int e = threadIdx.x; e < nh * dv; e += blockDim.x) {
    const int h = e / dv, i = e - h * dv;
    float v = 0.f;
    if (!pad) {
      v = kf_load(o, ((size_t)t * nh + h) * D + i);
      if (g) v *= 1.f / (1.f + expf(-g[(size_t)t * ld + gcol0 + h]));
      v *= scale;
    }
    kf_store(out, (size_t)t * ldo + ocol0 + e, v);
  }
}

// Eight elements per thread (one 16-byte load of bfloat16), the gate computed once for them.
__global__ void head_gate_vec_kernel(const __nv_bfloat16* __restrict__ o, const float* __restrict__ g, int ld, int gcol0, int nh,
                                     int dv, int D, __nv_bfloat16* __restrict__ out, const int* __restrict__ row_req, int ldo,
                                     int ocol0, float scale) {
  kf_pdl_trigger();
  kf_pdl_wait();
  const int t = blockIdx.x;
  const bool pad = row_req[t] < 0;
  for (int e = threadIdx.x * 8; e < nh * dv; e += blockDim.x * 8) {
    const int h = e / dv, i = e - h * dv;
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if (!pad) {
      raw = *reinterpret_cast<const uint4*>(o + ((size_t)t * nh + h) * D + i);
      if (g || scale != 1.f) {
        const float s = (g ? 1.f / (1.f + expf(-g[(size_t)t * ld + gcol0 + h])) : 1.f) * scale;
        __nv_bfloat162* pr = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = __bfloat1622float2(pr[k]);
          pr[k] = __floats2bfloat162_rn(f.x * s, f.y * s);
        }
      }
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * ldo + ocol0 + e) = raw;
  }
}

KF_API int kf_head_gate(const void* o, const float* g, int ld, int gcol0, int nh, int dv, int D, void* out, int dtype,
                        const int* row_req, int T, int ldo, int ocol0, float scale, cudaStream_t stream) {
  if (T <= 0) return KF_OK;
  if (ldo <= 0) ldo = nh * dv;                  // rows of `out` hold the heads alone
  if (ocol0 < 0 || ocol0 + nh * dv > ldo) return KF_ERR_SIZE;
  const int threads = nh * dv >= 1024 ? 256 : 128;
  if (dtype == KF_BF16 && dv % 8 == 0 && D % 8 == 0 && ldo % 8 == 0 && ocol0 % 8 == 0 && (((uintptr_t)o | (uintptr_t)out) & 15) == 0) {
    kf_launch(head_gate_vec_kernel, dim3(T), dim3(nh * dv >= 2048 ? 256 : 128), 0, stream, (const __nv_bfloat16*)o, g, ld, gcol0, nh,
              dv, D, (__nv_bfloat16*)out, row_req, ldo, ocol0, scale);
    KF_CHECK_LAUNCH();
    return KF_OK;
  }
  if (dtype == KF_F32)
    kf_launch(head_gate_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)o, g, ld, gcol0, nh, dv, D, (float*)out, row_req, ldo, ocol0, scale);
  else if (dtype == KF_BF16)
    kf_launch(head_gate_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, (const __nv_bfloat16*)o, g, ld, gcol0, nh, dv, D,
              (__nv_bfloat16*)out, row_req, ldo, ocol0, scale);
  else
    return KF_ERR_DTYPE;
  KF_CHECK_LAUNCH();
  return KF_OK;
}
