// Decode attention of every query head over every value head (the attention kernels' `vsplit` = G, see KfHeadMap), for
// rows that are the only row of their request.
//
// The ordinary decode kernels serve this case with one block per (key head, value head) pair, which computes the scores of
// a key head once per value head and reads every key and every value G times.  Here one block owns up to 16 query heads of
// a row (a tile of the heads) and ALL value heads, so scores and softmax are computed once:
//   per tile of 16 keys:  S = Q K_a^T for every key head a the tile's heads belong to (warp w takes a = w, w + 4, ...; a
//   head's row of S is kept from the product with its own key head), exchanged through shared memory; every warp then
//   makes the same online-softmax step on the whole 16 x 16 tile and multiplies P with the value tiles of ITS value heads
//   (c = w, w + 4, ...), which it accumulates in registers.
// The keys' range of a row is cut into `n_splits` parts (grid.y); every block writes one record per (head, value head):
// D sums, the base-2 running maximum and the sum of weights; kf_attn_vs_merge_kernel combines the records.  Results
// are laid out as the other kernels lay them out: result head ((a G + c) r + i) for query head a r + i over value head c.
#include "common.cuh"
#include "mma_tiles.cuh"

namespace {

constexpr int VS_WARPS = 4;
constexpr int VS_KEYS = 16;                       // keys per tile
constexpr int VS_STAGES = 2;
#define VS_PSTRIDE(D) ((D) + 4)

template <int D, int CPW>                          // CPW: value heads per warp (G <= VS_WARPS * CPW)
__global__ void __launch_bounds__(VS_WARPS * 32)
attn_decode_vs_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ pages,
                      const int* __restrict__ items, const int* __restrict__ positions, const int* __restrict__ row_req,
                      const int* __restrict__ table, int table_stride, int page_size, int H, int G, int ga_max,
                      float scale, int window, int n_splits, float* __restrict__ partial, __nv_bfloat16* __restrict__ out) {
  using namespace kf_mma;
  kf_pdl_trigger();
  kf_pdl_wait();
  constexpr int CH = D / 8;
  constexpr int NT_O = D / 8;
  constexpr int KS_QK = D / 16;
  constexpr int PS = VS_PSTRIDE(D);
  constexpr int TILE = VS_KEYS * D;
  extern __shared__ __align__(128) uint8_t vs_smem[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(vs_smem);            // [16][D]
  __nv_bfloat16* sKV = sQ + 16 * D;                                          // [stage][ga_max key tiles, G value tiles][16][D]
  __shared__ float sS[16][VS_KEYS + 2];

  const int MT = (H + 15) >> 4;
  const int item = blockIdx.x / MT, mt = blockIdx.x - item * MT;
  const int split = blockIdx.y;
  const int t = items ? items[item] : item;
  const int req = row_req[t];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int r = H / G;                                                       // query heads per key/value head
  const int h0 = mt * 16;
  const int n_rows = min(16, H - h0);
  const int a_lo = h0 / r, a_hi = (h0 + n_rows - 1) / r;
  const int GA = a_hi - a_lo + 1;                                            // key heads this tile of heads needs
  const int nhw = H * G;
  if (req < 0) {                                                             // a padding row: zeros (the merge writes them when there are splits)
    if (n_splits == 1)
      for (int e = tid; e < n_rows * G * D; e += blockDim.x) {
        const int i = e % D, c = (e / D) % G, h = h0 + e / (D * G);
        out[((size_t)t * nhw + ((h / r) * G + c) * r + h % r) * D + i] = __float2bfloat16_rn(0.f);
      }
    return;
  }
  const int pos = positions[t];
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int n_keys = pos + 1 - lo;
  int per = (n_keys + n_splits - 1) / n_splits;
  per = (per + 63) & ~63;
  const int k_begin = lo + split * per;
  const int k_end = min(pos + 1, k_begin + per);
  const int n_tiles = k_end > k_begin ? (k_end - k_begin + VS_KEYS - 1) / VS_KEYS : 0;
  const int* tab = table + (size_t)req * table_stride;
  const size_t head_stride = (size_t)page_size * D;
  const int stage_tiles = ga_max + G;

  // tile kt of the block's keys into stage kt % 2: the key tiles of heads a_lo .. a_hi, then the value tiles of all heads
  auto load_tile = [&](int kt) {
    __nv_bfloat16* dst0 = sKV + (size_t)(kt % VS_STAGES) * stage_tiles * TILE;
    const int j0 = k_begin + kt * VS_KEYS;
    // a thread owns (key row, 16-byte chunk) pairs: one look-up of the row's page, then that chunk of every head's tile
    for (int pc = tid; pc < VS_KEYS * CH; pc += VS_WARPS * 32) {
      const int row = pc / CH, c = pc - row * CH;
      const int j = j0 + row;
      bool ok = j < k_end;
      int page = 0;
      if (ok) { page = tab[j / page_size]; ok = page >= 0; }
      const __nv_bfloat16* base = pages + ((size_t)(ok ? page : 0) * 2 * G) * head_stride + (size_t)(ok ? j % page_size : 0) * D + c * 8;
      for (int ai = 0; ai < GA; ++ai)
        cp_async16(tile_ptr<D>(dst0 + (size_t)ai * TILE, row, c), base + (size_t)(a_lo + ai) * head_stride, ok);
      for (int cv = 0; cv < G; ++cv)
        cp_async16(tile_ptr<D>(dst0 + (size_t)(ga_max + cv) * TILE, row, c), base + (size_t)(G + cv) * head_stride, ok);
    }
  };

  if (n_tiles > 0) load_tile(0);
  cp_async_commit();
  // ---- Q: the tile's heads as rows, rows past the last head zero -------------------------------------------------------
  for (int idx = tid; idx < 16 * CH; idx += blockDim.x) {
    const int row = idx / CH, c = idx - row * CH;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < n_rows) v = *reinterpret_cast<const uint4*>(q + ((size_t)t * H + h0 + row) * D + c * 8);
    *reinterpret_cast<uint4*>(tile_ptr<D>(sQ, row, c)) = v;
  }
  for (int e = tid; e < 16 * (VS_KEYS + 2); e += blockDim.x) (&sS[0][0])[e] = 0.f;
  __syncthreads();
  uint32_t qf[KS_QK][4];
#pragma unroll
  for (int ks = 0; ks < KS_QK; ++ks) ldmatrix_x4(qf[ks], tile_ptr<D>(sQ, lane & 15, ks * 2 + (lane >> 4)));

  float o_acc[CPW][NT_O][4];
#pragma unroll
  for (int ci = 0; ci < CPW; ++ci)
#pragma unroll
    for (int n = 0; n < NT_O; ++n) o_acc[ci][n][0] = o_acc[ci][n][1] = o_acc[ci][n][2] = o_acc[ci][n][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  // which key head each of this thread's two rows (g and g + 8) belongs to; -1 for rows past the last head
  int row_a[2];
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) row_a[rr] = (g + 8 * rr < n_rows) ? (h0 + g + 8 * rr) / r : -1;

  for (int kt = 0; kt < n_tiles; ++kt) {
    __syncthreads();                                              // everyone is done with tile kt - 1: its stage and sS are free
    if (kt + 1 < n_tiles) load_tile(kt + 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();                                              // tile kt has landed for every thread
    const __nv_bfloat16* st = sKV + (size_t)(kt % VS_STAGES) * stage_tiles * TILE;
    const int j0 = k_begin + kt * VS_KEYS;
    // ---- scores: this warp's key heads; a row keeps the product with its own key head ---------------------------------
    for (int ai = warp; ai < GA; ai += VS_WARPS) {
      const __nv_bfloat16* k_s = st + (size_t)ai * TILE;
      float s_acc[2][4], s_odd[2][4];
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        s_acc[n][0] = s_acc[n][1] = s_acc[n][2] = s_acc[n][3] = 0.f;
        s_odd[n][0] = s_odd[n][1] = s_odd[n][2] = s_odd[n][3] = 0.f;
      }
#pragma unroll
      for (int ks = 0; ks < KS_QK; ++ks) {
        uint32_t b[4];
        ldmatrix_x4(b, tile_ptr<D>(const_cast<__nv_bfloat16*>(k_s), (lane & 7) + ((lane >> 4) << 3), ks * 2 + ((lane >> 3) & 1)));
        if (ks & 1) {
          mma_bf16(s_odd[0], qf[ks], b[0], b[1]);
          mma_bf16(s_odd[1], qf[ks], b[2], b[3]);
        } else {
          mma_bf16(s_acc[0], qf[ks], b[0], b[1]);
          mma_bf16(s_acc[1], qf[ks], b[2], b[3]);
        }
      }
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        if (row_a[rr] == a_lo + ai) {
#pragma unroll
          for (int n = 0; n < 2; ++n) {
            sS[g + 8 * rr][n * 8 + tq * 2] = s_acc[n][2 * rr] + s_odd[n][2 * rr];
            sS[g + 8 * rr][n * 8 + tq * 2 + 1] = s_acc[n][2 * rr + 1] + s_odd[n][2 * rr + 1];
          }
        }
      }
    }
    __syncthreads();                                              // the whole 16 x 16 tile of scores is in sS
    // ---- the online-softmax step, the same in every warp ---------------------------------------------------------------
    float p[2][4];
    float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
    for (int n = 0; n < 2; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int rr = e >> 1;
        const int j = j0 + n * 8 + tq * 2 + (e & 1);
        float s = sS[g + 8 * rr][n * 8 + tq * 2 + (e & 1)] * scale;
        s = (j < k_end) ? s * LOG2E : -INFINITY;
        p[n][e] = s;
        m_new[rr] = fmaxf(m_new[rr], s);
      }
    }
    float corr[2];
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      m_new[rr] = fmaxf(m_new[rr], __shfl_xor_sync(0xffffffffu, m_new[rr], 1));
      m_new[rr] = fmaxf(m_new[rr], __shfl_xor_sync(0xffffffffu, m_new[rr], 2));
      corr[rr] = (m_new[rr] == -INFINITY) ? 1.f : exp2f(m_run[rr] - m_new[rr]);
      m_run[rr] = m_new[rr];
    }
    float l_add[2] = {0.f, 0.f};
#pragma unroll
    for (int n = 0; n < 2; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int rr = e >> 1;
        const float w = (m_new[rr] == -INFINITY) ? 0.f : exp2f(p[n][e] - m_new[rr]);
        p[n][e] = w;
        l_add[rr] += w;
      }
    }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) l_run[rr] = l_run[rr] * corr[rr] + l_add[rr];
    uint32_t a[4];
    a[0] = pack_bf16(p[0][0], p[0][1]);
    a[1] = pack_bf16(p[0][2], p[0][3]);
    a[2] = pack_bf16(p[1][0], p[1][1]);
    a[3] = pack_bf16(p[1][2], p[1][3]);
    // ---- P times the value tiles of this warp's value heads --------------------------------------------------------------
#pragma unroll
    for (int ci = 0; ci < CPW; ++ci) {
      const int c = warp + ci * VS_WARPS;
      if (c < G) {
        const __nv_bfloat16* v_s = st + (size_t)(ga_max + c) * TILE;
#pragma unroll
        for (int n = 0; n < NT_O; ++n) {
          o_acc[ci][n][0] *= corr[0]; o_acc[ci][n][1] *= corr[0];
          o_acc[ci][n][2] *= corr[1]; o_acc[ci][n][3] *= corr[1];
        }
#pragma unroll
        for (int np = 0; np < NT_O / 2; ++np) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, tile_ptr<D>(const_cast<__nv_bfloat16*>(v_s), (lane & 7) + (((lane >> 3) & 1) << 3), np * 2 + (lane >> 4)));
          mma_bf16(o_acc[ci][2 * np], a, b[0], b[1]);
          mma_bf16(o_acc[ci][2 * np + 1], a, b[2], b[3]);
        }
      }
    }
  }
  cp_async_wait<0>();
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    l_run[rr] += __shfl_xor_sync(0xffffffffu, l_run[rr], 1);
    l_run[rr] += __shfl_xor_sync(0xffffffffu, l_run[rr], 2);
  }
  // ---- one record per (head, value head), or the result itself when the keys were not cut ------------------------------
#pragma unroll
  for (int ci = 0; ci < CPW; ++ci) {
    const int c = warp + ci * VS_WARPS;
    if (c >= G) continue;
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      const int row = g + 8 * rr;
      if (row >= n_rows) continue;
      const int h = h0 + row;
      const size_t wide = (size_t)t * nhw + ((h / r) * G + c) * r + h % r;
      if (n_splits == 1) {
        const float inv = l_run[rr] > 0.f ? 1.f / l_run[rr] : 0.f;
        __nv_bfloat16* dst = out + wide * D;
#pragma unroll
        for (int n = 0; n < NT_O; ++n)
          *reinterpret_cast<uint32_t*>(dst + n * 8 + tq * 2) = pack_bf16(o_acc[ci][n][2 * rr] * inv, o_acc[ci][n][2 * rr + 1] * inv);
      } else {
        float* rec = partial + (wide * n_splits + split) * PS;
#pragma unroll
        for (int n = 0; n < NT_O; ++n)
          *reinterpret_cast<float2*>(rec + n * 8 + tq * 2) = make_float2(o_acc[ci][n][2 * rr], o_acc[ci][n][2 * rr + 1]);
        if (tq == 0) { rec[D] = m_run[rr]; rec[D + 1] = l_run[rr]; }
      }
    }
  }
}

// One warp per (row of the step, result head): the records of the head's splits into the result.
template <int D>
__global__ void __launch_bounds__(128)
kf_attn_vs_merge_kernel(const float* __restrict__ partial, const int* __restrict__ items, int n_items,
                        const int* __restrict__ row_req, int nhw, int n_splits, __nv_bfloat16* __restrict__ out) {
  kf_pdl_trigger();
  kf_pdl_wait();
  constexpr int PS = VS_PSTRIDE(D);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long w = (long)blockIdx.x * 4 + warp;
  if (w >= (long)n_items * nhw) return;
  const int item = (int)(w / nhw), head = (int)(w - (long)item * nhw);
  const int t = items ? items[item] : item;
  __nv_bfloat16* dst = out + ((size_t)t * nhw + head) * D;
  if (row_req[t] < 0) {
    for (int i = lane; i < D; i += 32) dst[i] = __float2bfloat16_rn(0.f);
    return;
  }
  const float* rec0 = partial + ((size_t)t * nhw + head) * n_splits * PS;
  // lane s holds the statistics of parts s and s + 32 (at most 64 parts); both loads are in flight together
  const bool in0 = lane < n_splits, in1 = lane + 32 < n_splits;
  const float2 st0 = in0 ? __ldcg(reinterpret_cast<const float2*>(rec0 + (size_t)lane * PS + D)) : make_float2(-INFINITY, 0.f);
  const float2 st1 = in1 ? __ldcg(reinterpret_cast<const float2*>(rec0 + (size_t)(lane + 32) * PS + D)) : make_float2(-INFINITY, 0.f);
  const float m = kf_warp_max(fmaxf(st0.x, st1.x));
  float w0 = (st0.x == -INFINITY) ? 0.f : exp2f(st0.x - m);
  float w1 = (st1.x == -INFINITY) ? 0.f : exp2f(st1.x - m);
  const float l = kf_warp_sum(st0.y * w0 + st1.y * w1);
  const float inv = l > 0.f ? 1.f / l : 0.f;
  w0 *= inv, w1 *= inv;                                          // the weight of each part's sums in the result
  for (int base = 0; base < D / 4; base += 32) {                  // every lane walks the loop: the shuffles below need them all
    const int i4 = base + lane;
    const bool mine = i4 < D / 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int sp = 0; sp < n_splits; sp += 16) {
      float4 v[16];
#pragma unroll
      for (int u = 0; u < 16; ++u)
        v[u] = (mine && sp + u < n_splits) ? __ldcg(reinterpret_cast<const float4*>(rec0 + (size_t)(sp + u) * PS + i4 * 4))
                                           : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const int s_ = sp + u;                                    // the same in every lane
        const float c = __shfl_sync(0xffffffffu, s_ < 32 ? w0 : w1, s_ & 31);
        acc.x += v[u].x * c; acc.y += v[u].y * c; acc.z += v[u].z * c; acc.w += v[u].w * c;
      }
    }
    if (mine) {
      const __nv_bfloat162 a = __floats2bfloat162_rn(acc.x, acc.y), b2 = __floats2bfloat162_rn(acc.z, acc.w);
      uint2 packed;
      packed.x = *reinterpret_cast<const uint32_t*>(&a);
      packed.y = *reinterpret_cast<const uint32_t*>(&b2);
      *reinterpret_cast<uint2*>(dst + i4 * 4) = packed;
    }
  }
}

// The most key heads a tile of 16 query heads needs.
int vs_ga_max(int H, int G) {
  const int r = H / G;
  int best = 1;
  for (int h0 = 0; h0 < H; h0 += 16) {
    const int last = (h0 + 15 < H ? h0 + 15 : H - 1);
    const int ga = last / r - h0 / r + 1;
    if (ga > best) best = ga;
  }
  return best;
}

size_t vs_smem_bytes(int H, int G, int d) {
  return ((size_t)16 * d + (size_t)VS_STAGES * (vs_ga_max(H, G) + G) * VS_KEYS * d) * 2;
}

template <int D, int CPW>
int vs_launch(const void* q, void* out, const void* pages, const int* items, int n_items, const int* positions,
              const int* row_req, const int* table, int table_stride, int page_size, int H, int G, float scale, int window,
              int n_splits, float* partial, cudaStream_t stream) {
  const size_t smem = vs_smem_bytes(H, G, D);
  static size_t configured = 0;
  if (smem > configured) {
    if (cudaFuncSetAttribute(attn_decode_vs_kernel<D, CPW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      kf_record_cuda_error(cudaGetLastError());
      return KF_ERR_SETUP;
    }
    configured = smem;
  }
  const int MT = (H + 15) / 16;
  kf_launch(attn_decode_vs_kernel<D, CPW>, dim3(n_items * MT, n_splits), dim3(VS_WARPS * 32), smem, stream,
            (const __nv_bfloat16*)q, (const __nv_bfloat16*)pages, items, positions, row_req, table, table_stride, page_size, H, G,
            vs_ga_max(H, G), scale, window, n_splits, partial, (__nv_bfloat16*)out);
  KF_CHECK_LAUNCH();
  if (n_splits > 1) {
    const long warps = (long)n_items * H * G;
    kf_launch(kf_attn_vs_merge_kernel<D>, dim3((unsigned)((warps + 3) / 4)), dim3(128), 0, stream, (const float*)partial, items,
              n_items, row_req, H * G, n_splits, (__nv_bfloat16*)out);
    KF_CHECK_LAUNCH();
  }
  return KF_OK;
}

}  // namespace

// Whether the kernel takes these sizes (bfloat16, no softcap), and into how many parts it cuts a row's keys.  H query
// heads, G key/value heads of d elements.  KF_OK, or KF_ERR_SIZE when the ordinary decode kernels must do the work.
KF_API int kf_attention_decode_vs_plan(int n_items, int H, int G, int d, int max_keys, int* splits_out) {
  if (n_items < 1 || G < 1 || H % G || G > 2 * VS_WARPS) return KF_ERR_SIZE;
  if (!(d == 16 || d == 32 || d == 64 || d == 128 || d == 256)) return KF_ERR_SIZE;
  const int cpw = (G + VS_WARPS - 1) / VS_WARPS;
  if (cpw * d > 256) return KF_ERR_SIZE;                        // value accumulators of a warp: cpw * d / 2 registers per thread
  const size_t smem = vs_smem_bytes(H, G, d);
  if (smem > 200 * 1024) return KF_ERR_SIZE;
  long per_sm = (long)(220 * 1024 / (smem + 2048));
  if (per_sm > 4) per_sm = 4;
  if (per_sm < 1) per_sm = 1;
  const long blocks = (long)n_items * ((H + 15) / 16);
  int splits = (int)((kf_sm_count() * per_sm) / blocks);
  const int by_len = (max_keys + 127) / 128;                    // at least eight tiles of keys per part
  if (splits > by_len) splits = by_len;
  if (splits > 64) splits = 64;
  if (splits < 1) splits = 1;
  *splits_out = splits;
  return KF_OK;
}

// q: [T, H*d] bfloat16; out: [T, H*G*d]; pages of G heads.  partial: T * H * G * n_splits * (d + 4) floats when n_splits > 1.
// Launches the kernel and, when the keys are cut, the merge (two launches).
KF_API int kf_attention_decode_vs(const void* q, void* out, const void* pages, const int* items, int n_items,
                                  const int* positions, const int* row_req, const int* table, int table_stride, int page_size,
                                  int H, int G, int d, float scale, int window, int n_splits, float* partial,
                                  cudaStream_t stream) {
  if (n_items <= 0) return KF_OK;
  int planned = 0;
  if (kf_attention_decode_vs_plan(n_items, H, G, d, 1 << 20, &planned) != KF_OK || page_size < 1) return KF_ERR_SIZE;
  if (n_splits < 1 || n_splits > 64 || (n_splits > 1 && !partial)) return KF_ERR_SIZE;
  const int cpw = (G + VS_WARPS - 1) / VS_WARPS;
#define KF_ARGS q, out, pages, items, n_items, positions, row_req, table, table_stride, page_size, H, G, scale, window, n_splits, partial, stream
  if (cpw == 1) {
    switch (d) {
      case 16: return vs_launch<16, 1>(KF_ARGS);
      case 32: return vs_launch<32, 1>(KF_ARGS);
      case 64: return vs_launch<64, 1>(KF_ARGS);
      case 128: return vs_launch<128, 1>(KF_ARGS);
      case 256: return vs_launch<256, 1>(KF_ARGS);
    }
  } else {
    switch (d) {
      case 16: return vs_launch<16, 2>(KF_ARGS);
      case 32: return vs_launch<32, 2>(KF_ARGS);
      case 64: return vs_launch<64, 2>(KF_ARGS);
      case 128: return vs_launch<128, 2>(KF_ARGS);
    }
  }
#undef KF_ARGS
  return KF_ERR_SIZE;
}
