// Attention whose softmax weights are mixed across heads after the softmax ("talking heads"), served by the ordinary
// attention kernels.
//
// With H query heads, G key/value heads, r = H / G, and a mixing matrix M [H, H]:
//   a_g(i, .) = softmax over the visible keys of head g's scores            (each head's own weights)
//   b_h(i, j) = sum_g M[h, g] a_g(i, j)                                       (mixed weights)
//   out_h(i)  = sum_j b_h(i, j) v_(h / r)(j)  =  sum_g M[h, g] * O[g, h / r](i),   O[g, c] = sum_j a_g(., j) v_c(j).
// O[g, c] is plain attention of query head g over the keys of its own key head and the values of value head c, so the
// attention kernels produce H * G result heads from H query heads and G stored heads (their `vsplit` = G, see KfHeadMap):
// result head ((ck * G + cv) * r + i) is query head g = ck * r + i over the values of head cv.
//
// kf_rotate_norm_append: from the 32-bit q|k|v projection to the attention's operands.  Per head of q and k: the first
//   `rot` elements are turned in pairs (i, i + rot/2) by the step's cos/sin table times `mag`, then (when `unit_norm`) the
//   head is divided by sqrt(mean(head^2) + eps); v passes as it is.  q goes to q_out, k and v to the token's place in the
//   request's pages.  Heads use D elements in q and pages, tails zero.
// kf_head_mix_gate: out[t, h * dv + e] = gate(t, h * dv + e) * sum_g M[h, g] * o[t, wide(g, h / r), e], sums in 32-bit in
//   ascending g, gate = sigmoid of a column range of a 32-bit matrix (null: no gate).  Without M (null) it is the gate
//   and the packing alone.
// Everything is computed in 32-bit, only the stores round.
#include "common.cuh"

constexpr int HM_MAX_D = 256;
constexpr int HM_WARPS = 4;

__device__ __forceinline__ void hm_store4(float* p, const float* v) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
__device__ __forceinline__ void hm_store4(__nv_bfloat16* p, const float* v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 x;
  x.x = *reinterpret_cast<const uint32_t*>(&a), x.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = x;
}

// One warp per (row, head of q, k or v).  W = 4: a lane holds 4 neighbouring elements per 128 (16-byte loads, 8- or 16-byte
// stores; head sizes and row starts must be multiples of four elements); W = 1: element lane + 32 k, any sizes.  The head is
// staged in shared memory either way, so that a lane can read its elements' rotation partners.
template <typename TQ, typename TKV, int W>
__global__ void __launch_bounds__(HM_WARPS * 32)
rotate_norm_append_kernel(const float* __restrict__ in, int ld, int col0, const float* __restrict__ cos_t,
                          const float* __restrict__ sin_t, int rot, float mag, int unit_norm, float eps, int nh, int nkv,
                          int dk, int dv, int D, const int* __restrict__ positions,
                          const int* __restrict__ row_req, const int* __restrict__ block_table, int table_stride,
                          int page_size, TKV* __restrict__ pages, TQ* __restrict__ q_out, int write_kv, int T) {
  kf_pdl_trigger();
  kf_pdl_wait();
  constexpr int NK = HM_MAX_D / (32 * W);                   // groups of W elements per lane
  __shared__ __align__(16) float hs[HM_WARPS][HM_MAX_D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slots = nh + 2 * nkv;
  const long item = (long)blockIdx.x * HM_WARPS + warp;
  if (item >= (long)T * slots) return;                      // whole warps leave; only __syncwarp below
  const int t = (int)(item / slots), hslot = (int)(item - (long)t * slots);
  const int req = row_req[t];
  const int kind = hslot < nh ? 0 : (hslot < nh + nkv ? 1 : 2);            // query, key, value
  const int head = kind == 0 ? hslot : (kind == 1 ? hslot - nh : hslot - nh - nkv);
  float v[NK][W];
  if (req < 0) {                                            // padding row: zero queries, nothing filed
    if (kind == 0)
      for (int i = lane; i < D; i += 32) kf_store(q_out, ((size_t)t * nh + head) * D + i, 0.f);
    return;
  }
  if (kind != 0 && !write_kv) return;
  const int d = kind == 2 ? dv : dk;
  const float* src = in + (size_t)t * ld + col0 + (kind == 0 ? head * dk : (kind == 1 ? (nh + head) * dk : (nh + nkv) * dk + head * dv));
  float* x = hs[warp];
#pragma unroll
  for (int k = 0; k < NK; ++k) {
    const int i0 = (lane + 32 * k) * W;
    if (i0 < d) {
      if constexpr (W == 4) *reinterpret_cast<float4*>(x + i0) = *reinterpret_cast<const float4*>(src + i0);
      else x[i0] = src[i0];
    }
  }
  __syncwarp();
  const int half = rot >> 1;
  const float* c = cos_t + (size_t)t * half;
  const float* s = sin_t + (size_t)t * half;
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NK; ++k) {
#pragma unroll
    for (int e = 0; e < W; ++e) {
      const int i = (lane + 32 * k) * W + e;
      float y = 0.f;
      if (i < d) {
        y = x[i];
        if (kind != 2 && i < rot)
          y = i < half ? x[i] * (c[i] * mag) - x[i + half] * (s[i] * mag) : x[i] * (c[i - half] * mag) + x[i - half] * (s[i - half] * mag);
        ss = fmaf(y, y, ss);
      }
      v[k][e] = y;
    }
  }
  if (kind != 2 && unit_norm) {
    ss = kf_warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)d + eps);
#pragma unroll
    for (int k = 0; k < NK; ++k)
#pragma unroll
      for (int e = 0; e < W; ++e) v[k][e] *= inv;
  }
  int page = -1, in_page = 0;
  if (kind != 0) {
    const int pos = positions[t];
    page = block_table[(size_t)req * table_stride + pos / page_size];
    in_page = pos % page_size;
    if (page < 0) return;                                   // never for a reserved position; guards the store
  }
  auto put = [&](auto* o) {
#pragma unroll
    for (int k = 0; k < NK; ++k) {
      const int i0 = (lane + 32 * k) * W;
      if (i0 < D) {
        if constexpr (W == 4) hm_store4(o + i0, v[k]);
        else kf_store(o, i0, v[k][0]);
      }
    }
  };
  if (kind == 0) put(q_out + ((size_t)t * nh + head) * D);
  else put(pages + ((((size_t)page * 2 + (kind - 1)) * nkv + head) * page_size + in_page) * D);
}

KF_API int kf_rotate_norm_append(const float* in, int ld, int col0, const float* cos_t, const float* sin_t, int rot, float mag,
                                 int unit_norm, float eps, int nh, int nkv, int dk, int dv, int D,
                                 const int* positions, const int* row_req, const int* block_table, int table_stride,
                                 int page_size, void* pages, int kv_dtype, void* q_out, int q_dtype, int write_kv, int T,
                                 cudaStream_t stream) {
  if (T <= 0) return KF_OK;
  if (D > HM_MAX_D || dk > D || dv > D || dk < 1 || dv < 1 || rot > dk || (rot & 1) || nkv < 1 || nh % nkv) return KF_ERR_SIZE;
  if (rot > 0 && (!cos_t || !sin_t)) return KF_ERR_SIZE;
  const long n_work = (long)T * (nh + 2 * nkv);
  const dim3 grid((unsigned)((n_work + HM_WARPS - 1) / HM_WARPS));
  const bool by4 = dk % 4 == 0 && dv % 4 == 0 && D % 4 == 0 && ld % 4 == 0 && col0 % 4 == 0 && ((uintptr_t)in & 15) == 0 &&
                   ((uintptr_t)pages & 15) == 0 && ((uintptr_t)q_out & 15) == 0;
#define KF_GO1(TQ, TKV, W)                                                                                                \
  kf_launch(rotate_norm_append_kernel<TQ, TKV, W>, grid, dim3(HM_WARPS * 32), 0, stream, in, ld, col0, cos_t, sin_t, rot, mag, \
            unit_norm, eps, nh, nkv, dk, dv, D, positions, row_req, block_table, table_stride, page_size,           \
            (TKV*)pages, (TQ*)q_out, write_kv, T)
#define KF_GO(TQ, TKV) do { if (by4) KF_GO1(TQ, TKV, 4); else KF_GO1(TQ, TKV, 1); } while (0)
  if (q_dtype == KF_F32 && kv_dtype == KF_F32) KF_GO(float, float);
  else if (q_dtype == KF_BF16 && kv_dtype == KF_BF16) KF_GO(__nv_bfloat16, __nv_bfloat16);
  else return KF_ERR_DTYPE;
#undef KF_GO
#undef KF_GO1
  KF_CHECK_LAUNCH();
  return KF_OK;
}

constexpr int HG_THREADS = 128;
constexpr int HG_LOADS = 8;                                 // loads a thread has in flight
constexpr int HG_HEADS = 4;                                 // result heads a thread sums at a time

template <int VEC> struct HgVec { float v[VEC]; };
template <int VEC> __device__ __forceinline__ HgVec<VEC> hg_load(const float* p) {
  HgVec<VEC> r;
  if constexpr (VEC == 4) { const float4 x = *reinterpret_cast<const float4*>(p); r.v[0] = x.x, r.v[1] = x.y, r.v[2] = x.z, r.v[3] = x.w; }
  else { const float2 x = *reinterpret_cast<const float2*>(p); r.v[0] = x.x, r.v[1] = x.y; }
  return r;
}
template <int VEC> __device__ __forceinline__ HgVec<VEC> hg_load(const __nv_bfloat16* p) {
  HgVec<VEC> r;
  if constexpr (VEC == 4) {
    const uint2 x = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x.y));
    r.v[0] = a.x, r.v[1] = a.y, r.v[2] = b.x, r.v[3] = b.y;
  } else {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    r.v[0] = a.x, r.v[1] = a.y;
  }
  return r;
}
// The same elements as they lie in memory (converted when they are used, so that eight loads in flight cost few registers).
template <typename T, int VEC> struct HgRaw;
template <> struct HgRaw<float, 4> { float4 r; __device__ void load(const float* p) { r = *reinterpret_cast<const float4*>(p); }
  __device__ void get(float* v) const { v[0] = r.x, v[1] = r.y, v[2] = r.z, v[3] = r.w; } };
template <> struct HgRaw<float, 2> { float2 r; __device__ void load(const float* p) { r = *reinterpret_cast<const float2*>(p); }
  __device__ void get(float* v) const { v[0] = r.x, v[1] = r.y; } };
template <> struct HgRaw<__nv_bfloat16, 4> { uint2 r; __device__ void load(const __nv_bfloat16* p) { r = *reinterpret_cast<const uint2*>(p); }
  __device__ void get(float* v) const {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
    v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y; } };
template <> struct HgRaw<__nv_bfloat16, 2> { uint32_t r; __device__ void load(const __nv_bfloat16* p) { r = *reinterpret_cast<const uint32_t*>(p); }
  __device__ void get(float* v) const { const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r)); v[0] = a.x, v[1] = a.y; } };

__device__ __forceinline__ void hg_store4(float* p, const float* v) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
__device__ __forceinline__ void hg_store4(__nv_bfloat16* p, const float* v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 x;
  x.x = *reinterpret_cast<const uint32_t*>(&a), x.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = x;
}

// One thread per (row, value head c, VEC neighbouring elements): it reads those elements of every query head's result over
// value head c once and sums them into the r heads of c's group.  M sits in shared memory when it fits (else it is read
// through L1).  VEC = 4 needs rows whose starts and head sizes are multiples of four elements (16-byte gate loads and
// 8- or 16-byte stores); VEC = 2 takes every even D and any dv, with element-wise gate loads and stores.
template <typename TQ, typename TW, int VEC>
__global__ void __launch_bounds__(HG_THREADS, 5)
head_mix_gate_kernel(const TQ* __restrict__ o, const TW* __restrict__ mix, const float* __restrict__ g, int ld, int gcol0,
                     int nh, int nkv, int dv, int D, TQ* __restrict__ out, const int* __restrict__ row_req, int T,
                     int mix_in_smem) {
  kf_pdl_trigger();
  kf_pdl_wait();
  extern __shared__ float ms[];                             // the mixing matrix [nh, nh]
  if (mix && mix_in_smem) {
    for (int i = threadIdx.x; i < nh * nh; i += blockDim.x) ms[i] = kf_load(mix, i);
    __syncthreads();
  }
  const int per = nh / nkv;
  const int chunks = (dv + VEC - 1) / VEC;
  const int groups = mix ? nkv : nh;                        // without M every head is a group of its own
  const long item = (long)blockIdx.x * HG_THREADS + threadIdx.x;
  if (item >= (long)T * groups * chunks) return;
  const int ic = (int)(item % chunks);
  const int cv = (int)((item / chunks) % groups);
  const int t = (int)(item / ((long)chunks * groups));
  const int i = VEC * ic;
  const bool pad = row_req[t] < 0;
  auto put = [&](int h, float* a) {
    const size_t e = (size_t)h * dv + i;
    if constexpr (VEC == 4) {
      if (pad) a[0] = a[1] = a[2] = a[3] = 0.f;
      else if (g) {
        const HgVec<4> gr = hg_load<4>(g + (size_t)t * ld + gcol0 + e);
#pragma unroll
        for (int k = 0; k < 4; ++k) a[k] *= 1.f / (1.f + expf(-gr.v[k]));
      }
      hg_store4(out + (size_t)t * nh * dv + e, a);
    } else {
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        if (i + k < dv) {
          float x = pad ? 0.f : a[k];
          if (!pad && g) x *= 1.f / (1.f + expf(-g[(size_t)t * ld + gcol0 + e + k]));
          kf_store(out, (size_t)t * nh * dv + e + k, x);
        }
      }
    }
  };
  if (!mix) {
    HgVec<VEC> v = hg_load<VEC>(o + ((size_t)t * nh + cv) * D + i);
    put(cv, v.v);
    return;
  }
  const TQ* orow = o + (size_t)t * nh * nkv * D + i;
  for (int h0 = 0; h0 < per; h0 += HG_HEADS) {
    float acc[HG_HEADS][VEC];
#pragma unroll
    for (int j = 0; j < HG_HEADS; ++j)
#pragma unroll
      for (int k = 0; k < VEC; ++k) acc[j][k] = 0.f;
    if (!pad) {
      const int hn = min(HG_HEADS, per - h0);               // heads of this pass
      const int m0 = (cv * per + h0) * nh;                  // M[first head of the pass, 0]
      int kh = 0, q = 0;                                    // query head gq = kh * r + q, in ascending order
      for (int g0 = 0; g0 < nh; g0 += HG_LOADS) {
        HgRaw<TQ, VEC> raw[HG_LOADS];
#pragma unroll
        for (int u = 0; u < HG_LOADS; ++u) {                // the loads of eight query heads first, then their sums
          if (g0 + u < nh) {
            raw[u].load(orow + (size_t)((kh * nkv + cv) * per + q) * D);
            if (++q == per) q = 0, ++kh;
          }
        }
#pragma unroll
        for (int u = 0; u < HG_LOADS; ++u) {
          if (g0 + u < nh) {
            float v[VEC];
            raw[u].get(v);
#pragma unroll
            for (int j = 0; j < HG_HEADS; ++j) {
              const int mi = m0 + (j < hn ? j : 0) * nh + g0 + u;   // heads past the pass repeat its first: summed, never stored
              const float m = mix_in_smem ? ms[mi] : kf_load(mix, mi);
#pragma unroll
              for (int k = 0; k < VEC; ++k) acc[j][k] = fmaf(m, v[k], acc[j][k]);
            }
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < HG_HEADS; ++j)
      if (h0 + j < per) put(cv * per + h0 + j, acc[j]);
  }
}

KF_API int kf_head_mix_gate(const void* o, const void* mix, int w_dtype, const float* g, int ld, int gcol0, int nh, int nkv,
                            int dv, int D, void* out, int dtype, const int* row_req, int T, cudaStream_t stream) {
  if (T <= 0) return KF_OK;
  if (nkv < 1 || nh % nkv || dv > D || (D & 1)) return KF_ERR_SIZE;
  const size_t want = mix ? (size_t)nh * nh * sizeof(float) : 0;
  const int in_smem = want <= 40 * 1024;
  const size_t smem = in_smem ? want : 0;
  const bool by4 = dv % 4 == 0 && D % 4 == 0 && (!g || (ld % 4 == 0 && gcol0 % 4 == 0 && ((uintptr_t)g & 15) == 0)) &&
                   ((uintptr_t)o & 15) == 0 && ((uintptr_t)out & 15) == 0;
  const int vec = by4 ? 4 : 2;
  const long n_work = (long)T * (mix ? nkv : nh) * ((dv + vec - 1) / vec);
  const dim3 grid((unsigned)((n_work + HG_THREADS - 1) / HG_THREADS));
#define KF_GO2(TQ, TW, VEC)                                                                                          \
  kf_launch(head_mix_gate_kernel<TQ, TW, VEC>, grid, dim3(HG_THREADS), smem, stream, (const TQ*)o, (const TW*)mix, g, ld,  \
            gcol0, nh, nkv, dv, D, (TQ*)out, row_req, T, in_smem)
#define KF_GO(TQ, TW) do { if (by4) KF_GO2(TQ, TW, 4); else KF_GO2(TQ, TW, 2); } while (0)
  if (dtype == KF_F32 && w_dtype == KF_F32) KF_GO(float, float);
  else if (dtype == KF_BF16 && w_dtype == KF_BF16) KF_GO(__nv_bfloat16, __nv_bfloat16);
  else if (dtype == KF_BF16 && w_dtype == KF_F32) KF_GO(__nv_bfloat16, float);
  else if (dtype == KF_F32 && w_dtype == KF_BF16) KF_GO(float, __nv_bfloat16);
  else return KF_ERR_DTYPE;
#undef KF_GO
#undef KF_GO2
  KF_CHECK_LAUNCH();
  return KF_OK;
}
