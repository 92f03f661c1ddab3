// Products in groups, and the router of a mixture of experts.
//
// kf_grouped_linear:  out_g[r, n] = sum_k x_g[r, k] w_g[n, k]  for a set of groups g that each have their own weight
//   matrix, in 32-bit FMA accumulation, summed over k in ascending order by one thread (a row's result does not depend
//   on which other rows share the launch or the group).  Two ways to say which rows belong to which group:
//     * every group takes all T rows (grid z = group): the per-head maps of latent attention, where x_g and out_g are
//       column ranges of one matrix (x + g * x_gstride, row pitch ldx);
//     * a tile list (tile_group, tile_row0, tile_nrows, n_tiles on the device): the experts of a mixture, whose rows
//       are the (token, choice) pairs sorted by expert; `row_index` then names the source row of a sorted row
//       (row_index[r] / row_div), or the sorted row itself when absent.
//   gated = 1: w_g holds 2N rows (gate rows, then up rows) and out = act(gate, up) with the clamped form
//       g = min(gate, limit), u = clamp(up, -limit, limit), out = g * sigmoid(1.702 g) * (u + 1);
//   gated = 2: the same rows with out = gate * sigmoid(gate) * up.
//
// kf_moe_route: sigmoid scores (or, `softmax`, the softmax over all experts), a correction added for the choice only,
//   groups of neighbouring experts ranked by the sum of their two largest choice scores (or, `group_best` = 1, by their
//   largest), the best `keep` groups stay eligible, the `top` largest eligible choice scores win (lower index first
//   among equals); weights = the winners' uncorrected scores, divided by their sum + 1e-20 when `normalize`, times
//   `scale`.  One warp per token, everything 32-bit.
// kf_moe_plan: counts the pairs of every expert, lays the pairs out expert by expert (sorted_pair, inverse), and lists
//   the row tiles of every expert.  One block; the order inside an expert is whatever the atomics give, which no
//   result depends on (a pair's output row is computed from its own row alone).
// kf_moe_combine: y[t] = sum_j weight[t, j] * expert_out[inverse[t * top + j]] (+ shared[t]), j ascending; without
//   weights (null) every weight is one (mixtures whose weights went into the experts' inputs).
#include "mma_tiles.cuh"

constexpr int GM = 64, GN = 64, GK = 16;

struct KfGroupedArgs {
  const void* x; long ldx, x_gstride;
  const int* row_index; int row_div;
  const void* w; long w_gstride;
  void* out; long ldo, o_gstride;
  const int* tile_group; const int* tile_row0; const int* tile_nrows; const int* n_tiles;
  int T, N, K, gated;
  float limit;
  const float* row_scale;      // gated products: gate and up of sorted row r are multiplied by row_scale[row_index[r]] first
};

template <typename TX, typename TW, typename TO, int GATED>
__global__ void __launch_bounds__(256) grouped_simt_kernel(KfGroupedArgs p) {
  kf_pdl_trigger();
  kf_pdl_wait();
  __shared__ float xs[GK][GM + 4];
  __shared__ float ws[GK][GN + 4];
  __shared__ float us[GATED ? GK : 1][GN + 4];
  __shared__ int src_row[GM];
  int g, r0, nrows;
  if (p.tile_group) {
    const int ti = blockIdx.y;
    if (ti >= *p.n_tiles) return;
    g = p.tile_group[ti]; r0 = p.tile_row0[ti]; nrows = p.tile_nrows[ti];
  } else {
    g = blockIdx.z; r0 = blockIdx.y * GM; nrows = min(GM, p.T - r0);
  }
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int col0 = blockIdx.x * GN;
  const int N = p.N, K = p.K;
  if (tid < GM) src_row[tid] = tid < nrows ? (p.row_index ? p.row_index[r0 + tid] / p.row_div : r0 + tid) : -1;
  __syncthreads();
  const TX* x = (const TX*)p.x + (size_t)g * p.x_gstride;
  const TW* w = (const TW*)p.w + (size_t)g * p.w_gstride;
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  float acc[4][4], acu[GATED ? 4 : 1][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) { acc[i][j] = 0.f; if (GATED) acu[i][j] = 0.f; }
  for (int k0 = 0; k0 < K; k0 += GK) {
    {
      const int sr = src_row[lr];
      const TX* px = x + (size_t)(sr < 0 ? 0 : sr) * p.ldx + k0 + lk;
#pragma unroll
      for (int u = 0; u < 4; ++u) xs[lk + u][lr] = (sr >= 0 && k0 + lk + u < K) ? kf_load(px, u) : 0.f;
      const int c = col0 + lr;
      const TW* pw = w + (size_t)c * K + k0 + lk;
#pragma unroll
      for (int u = 0; u < 4; ++u) ws[lk + u][lr] = (c < N && k0 + lk + u < K) ? kf_load(pw, u) : 0.f;
      if (GATED) {
        const TW* pu = w + (size_t)(N + c) * K + k0 + lk;
#pragma unroll
        for (int u = 0; u < 4; ++u) us[lk + u][lr] = (c < N && k0 + lk + u < K) ? kf_load(pu, u) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < GK; ++k) {
      float a[4], b[4], bu[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) { b[j] = ws[k][tx * 4 + j]; if (GATED) bu[j] = us[k][tx * 4 + j]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
          if (GATED) acu[i][j] = fmaf(a[i], bu[j], acu[i][j]);
        }
    }
    __syncthreads();
  }
  TO* out = (TO*)p.out + (size_t)g * p.o_gstride;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty * 4 + i;
    if (r >= nrows) continue;
    const float rs = (GATED && p.row_scale) ? p.row_scale[p.row_index ? p.row_index[r0 + r] : r0 + r] : 1.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = col0 + tx * 4 + j;
      if (c >= N) continue;
      float v = acc[i][j] * rs;
      if (GATED) v = p.gated == 2 ? v / (1.f + expf(-v)) * (acu[i][j] * rs) : kf_clamped_swish(v, acu[i][j] * rs, p.limit);
      kf_store(out, (size_t)(r0 + r) * p.ldo + c, v);
    }
  }
}

// The same products on the tensor cores (mma.sync m16n8k16, bfloat16 operands, 32-bit accumulators) for bfloat16 weights:
// a block of eight warps owns 64 rows x 128 weight rows (gated: 64 gate rows and the 64 up rows of the same features, so
// that the warp that holds a gate value also holds its up value and the activation needs no exchange), K in slices of 32
// through a ring of three stages filled by 16-byte cp.async copies (32-bit rows are converted on their way into shared
// memory instead).  Shared rows are 40 elements (80 bytes) apart: the eight 16-byte rows of an ldmatrix fall into
// different banks.  A row's sums do not depend on the other rows of its tile.
constexpr int TM = 64, TN = 128, TK = 32, TSTAGES = 3, TLD = TK + 8;

template <typename TX, typename TO, int GATED>
__global__ void __launch_bounds__(256) grouped_mma_kernel(KfGroupedArgs p) {
  using namespace kf_mma;
  kf_pdl_trigger();
  kf_pdl_wait();
  __shared__ __align__(16) __nv_bfloat16 xs[TSTAGES][TM][TLD];
  __shared__ __align__(16) __nv_bfloat16 ws[TSTAGES][TN][TLD];
  __shared__ int src_row[TM];
  int g, r0, nrows;
  if (p.tile_group) {
    const int ti = blockIdx.y;
    if (ti >= *p.n_tiles) return;
    g = p.tile_group[ti]; r0 = p.tile_row0[ti]; nrows = p.tile_nrows[ti];
  } else {
    g = blockIdx.z; r0 = blockIdx.y * TM; nrows = min(TM, p.T - r0);
  }
  constexpr int NOUT = GATED ? TN / 2 : TN;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tig = lane & 3;
  const int wm = warp >> 2, wn = warp & 3;
  const int col0 = blockIdx.x * NOUT;
  const int N = p.N, K = p.K;
  if (tid < TM) src_row[tid] = tid < nrows ? (p.row_index ? p.row_index[r0 + tid] / p.row_div : r0 + tid) : -1;
  __syncthreads();
  const TX* x = (const TX*)p.x + (size_t)g * p.x_gstride;
  const __nv_bfloat16* w = (const __nv_bfloat16*)p.w + (size_t)g * p.w_gstride;

  auto load_stage = [&](int s, int k0) {
#pragma unroll
    for (int it = 0; it < 2; ++it) {                     // weights: 128 rows x 4 chunks of 8 elements
      const int idx = tid + it * 256, r = idx >> 2, c = idx & 3;
      const int feat = col0 + (GATED ? (r & 63) : r);
      const size_t wrow = GATED && r >= 64 ? (size_t)N + feat : (size_t)feat;
      const bool ok = feat < N && k0 + c * 8 < K;
      cp_async16(&ws[s][r][c * 8], w + (ok ? wrow * K + k0 + c * 8 : 0), ok);
    }
    const int r = tid >> 2, c = tid & 3, sr = src_row[r];
    if (sizeof(TX) == 2) {
      const bool ok = sr >= 0 && k0 + c * 8 < K;
      cp_async16(&xs[s][r][c * 8], (const __nv_bfloat16*)x + (ok ? (size_t)sr * p.ldx + k0 + c * 8 : 0), ok);
    } else {
      uint32_t v[4] = {0u, 0u, 0u, 0u};
      if (sr >= 0 && k0 + c * 8 < K) {                   // K is a multiple of 8: the chunk is whole
        const float* src = (const float*)x + (size_t)sr * p.ldx + k0 + c * 8;
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = pack_bf16(src[2 * u], src[2 * u + 1]);
      }
      *reinterpret_cast<uint4*>(&xs[s][r][c * 8]) = make_uint4(v[0], v[1], v[2], v[3]);
    }
  };

  float acc[2][4][4];
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[a][b][c] = 0.f;
  const int nk = (K + TK - 1) / TK;
#pragma unroll
  for (int s = 0; s < TSTAGES - 1; ++s) {
    if (s < nk) load_stage(s, s * TK);
    cp_async_commit();
  }
  // weight row (inside the tile) of this warp's n-tile nt
  int wrow_of[4];
#pragma unroll
  for (int nt = 0; nt < 4; ++nt) wrow_of[nt] = GATED ? (nt < 2 ? wn * 16 + nt * 8 : 64 + wn * 16 + (nt - 2) * 8) : wn * 32 + nt * 8;
  for (int kt = 0; kt < nk; ++kt) {
    cp_async_wait<TSTAGES - 2>();
    __syncthreads();
    if (kt + TSTAGES - 1 < nk) load_stage((kt + TSTAGES - 1) % TSTAGES, (kt + TSTAGES - 1) * TK);
    cp_async_commit();
    const int s = kt % TSTAGES;
#pragma unroll
    for (int kk = 0; kk < TK; kk += 16) {
      // fragments by ldmatrix: lane i names row i % 8 of 8 x 8 matrix i / 8.  A: matrices (rows 0-7, k 0-7), (rows 8-15, k 0-7),
      // (rows 0-7, k 8-15), (rows 8-15, k 8-15) are a0..a3; B from [n][k] rows: (n 0-7, k 0-7), (n 0-7, k 8-15) are b0, b1 of
      // one n-tile and (n 8-15, ...) those of the next.
      uint32_t a[2][4], b[4][2];
      const int lm = lane >> 3, lr = lane & 7;
#pragma unroll
      for (int mi = 0; mi < 2; ++mi)
        ldmatrix_x4(a[mi], &xs[s][wm * 32 + mi * 16 + (lm & 1) * 8 + lr][kk + (lm >> 1) * 8]);
#pragma unroll
      for (int np = 0; np < 2; ++np) {
        uint32_t r[4];
        ldmatrix_x4(r, &ws[s][wrow_of[2 * np] + (lm >> 1) * 8 + lr][kk + (lm & 1) * 8]);
        b[2 * np][0] = r[0]; b[2 * np][1] = r[1]; b[2 * np + 1][0] = r[2]; b[2 * np + 1][1] = r[3];
      }
#pragma unroll
      for (int mi = 0; mi < 2; ++mi)
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) mma_bf16(acc[mi][nt], a[mi], b[nt][0], b[nt][1]);
    }
  }
  cp_async_wait<0>();
  TO* out = (TO*)p.out + (size_t)g * p.o_gstride;
#pragma unroll
  for (int mi = 0; mi < 2; ++mi)
#pragma unroll
    for (int nt = 0; nt < (GATED ? 2 : 4); ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = wm * 32 + mi * 16 + gid + (i >= 2 ? 8 : 0);
        const int c = col0 + (GATED ? wn * 16 + nt * 8 : wn * 32 + nt * 8) + 2 * tig + (i & 1);
        if (r >= nrows || c >= N) continue;
        const float rs = (GATED && p.row_scale) ? p.row_scale[p.row_index ? p.row_index[r0 + r] : r0 + r] : 1.f;
        const float ga = acc[mi][nt][i] * rs, up = GATED ? acc[mi][nt + 2][i] * rs : 0.f;
        const float v = !GATED ? acc[mi][nt][i]
                        : (p.gated == 2 ? ga / (1.f + expf(-ga)) * up : kf_clamped_swish(ga, up, p.limit));
        kf_store(out, (size_t)(r0 + r) * p.ldo + c, v);
      }
}

template <typename TX, typename TO>
static int grouped_mma_go(const KfGroupedArgs& p, int max_tiles, int n_groups, cudaStream_t s) {
  const int nout = p.gated ? TN / 2 : TN;
  const dim3 grid(kf_ceil_div(p.N, nout), p.tile_group ? max_tiles : kf_ceil_div(p.T, TM), p.tile_group ? 1 : n_groups);
  if (p.gated) kf_launch(grouped_mma_kernel<TX, TO, 1>, grid, dim3(256), 0, s, p);
  else kf_launch(grouped_mma_kernel<TX, TO, 0>, grid, dim3(256), 0, s, p);
  KF_CHECK_LAUNCH();
  return KF_OK;
}

static int g_grouped_tensor_cores = 1;
KF_API void kf_grouped_use_tensor_cores(int on) { g_grouped_tensor_cores = on; }

template <typename TX, typename TW, typename TO>
static int grouped_go(const KfGroupedArgs& p, dim3 grid, cudaStream_t s) {
  if (p.gated) kf_launch(grouped_simt_kernel<TX, TW, TO, 1>, grid, dim3(256), 0, s, p);
  else kf_launch(grouped_simt_kernel<TX, TW, TO, 0>, grid, dim3(256), 0, s, p);
  KF_CHECK_LAUNCH();
  return KF_OK;
}

// x_off / o_off: element offsets of the first group's first column inside x / out.  n_groups and T describe the
// all-rows form; with a tile list, max_tiles bounds the grid and *n_tiles says how many tiles are real.
KF_API int kf_grouped_linear(const void* x, int x_dtype, long x_off, long ldx, long x_gstride, const int* row_index, int row_div,
                             const void* w, int w_dtype, long w_gstride, void* out, int out_dtype, long o_off, long ldo,
                             long o_gstride, const int* tile_group, const int* tile_row0, const int* tile_nrows,
                             const int* n_tiles, int max_tiles, int n_groups, int T, int N, int K, int gated, float limit,
                             const float* row_scale, cudaStream_t stream) {
  if (N <= 0 || (tile_group ? max_tiles <= 0 : (T <= 0 || n_groups <= 0))) return KF_OK;
  if (K <= 0) return KF_ERR_SIZE;
  const size_t xe = x_dtype == KF_F32 ? 4 : 2, oe = out_dtype == KF_F32 ? 4 : 2;
  KfGroupedArgs p{(const char*)x + x_off * xe, ldx, x_gstride, row_index, row_div > 0 ? row_div : 1, w, w_gstride,
                  (char*)out + o_off * oe, ldo, o_gstride, tile_group, tile_row0, tile_nrows, n_tiles, T, N, K, gated, limit, row_scale};
  // bfloat16 weights whose rows, groups and bases fall on 16-byte boundaries run on the tensor cores; their row tiles are
  // the plan's 64 rows (GM == TM)
  const bool w_ok = w_dtype == KF_BF16 && K % 8 == 0 && w_gstride % 8 == 0 && ((uintptr_t)w & 15) == 0;
  const bool x_ok = x_dtype == KF_F32 || (ldx % 8 == 0 && x_gstride % 8 == 0 && x_off % 8 == 0 && ((uintptr_t)x & 15) == 0);
  if (g_grouped_tensor_cores && w_ok && x_ok) {
    if (x_dtype == KF_BF16 && out_dtype == KF_BF16) return grouped_mma_go<__nv_bfloat16, __nv_bfloat16>(p, max_tiles, n_groups, stream);
    if (x_dtype == KF_BF16 && out_dtype == KF_F32) return grouped_mma_go<__nv_bfloat16, float>(p, max_tiles, n_groups, stream);
    if (x_dtype == KF_F32 && out_dtype == KF_BF16) return grouped_mma_go<float, __nv_bfloat16>(p, max_tiles, n_groups, stream);
    if (x_dtype == KF_F32 && out_dtype == KF_F32) return grouped_mma_go<float, float>(p, max_tiles, n_groups, stream);
  }
  const dim3 grid(kf_ceil_div(N, GN), tile_group ? max_tiles : kf_ceil_div(T, GM), tile_group ? 1 : n_groups);
#define KF_CASE(XD, WD, OD, TX, TW, TO) \
  if (x_dtype == XD && w_dtype == WD && out_dtype == OD) return grouped_go<TX, TW, TO>(p, grid, stream)
  KF_CASE(KF_F32, KF_F32, KF_F32, float, float, float);
  KF_CASE(KF_F32, KF_BF16, KF_BF16, float, __nv_bfloat16, __nv_bfloat16);
  KF_CASE(KF_F32, KF_BF16, KF_F32, float, __nv_bfloat16, float);
  KF_CASE(KF_BF16, KF_BF16, KF_BF16, __nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
  KF_CASE(KF_BF16, KF_BF16, KF_F32, __nv_bfloat16, __nv_bfloat16, float);
  KF_CASE(KF_BF16, KF_F32, KF_F32, __nv_bfloat16, float, float);
  KF_CASE(KF_F32, KF_F32, KF_BF16, float, float, __nv_bfloat16);
#undef KF_CASE
  return KF_ERR_DTYPE;
}

// ---- the router ------------------------------------------------------------------------------------------------------

constexpr int KF_MOE_MAX_EXPERTS = 1024;

template <typename TW>
__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ logits, const TW* __restrict__ correction,
                                                        int T, int E, int G, int keep, int top, float scale, int softmax,
                                                        int group_best, int normalize,
                                                        int* __restrict__ ids, float* __restrict__ weights) {
  kf_pdl_trigger();
  kf_pdl_wait();
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= T) return;
  float* score = sm + (size_t)warp * (2 * E + G);      // uncorrected sigmoid
  float* choice = score + E;                           // corrected; -inf when not eligible or already taken
  float* gscore = choice + E;
  const float NEG = -INFINITY;
  float zmax = NEG, zsum = 0.f;
  if (softmax) {
    for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, logits[(size_t)t * E + e]);
    zmax = kf_warp_max(zmax);
    for (int e = lane; e < E; e += 32) zsum += expf(logits[(size_t)t * E + e] - zmax);
    zsum = kf_warp_sum(zsum);
  }
  for (int e = lane; e < E; e += 32) {
    const float z = logits[(size_t)t * E + e];
    const float s = softmax ? expf(z - zmax) / zsum : 1.f / (1.f + expf(-z));
    score[e] = s;
    // sigmoid scores without a correction and without groups rank as their logits do, and the logits do not run into
    // one another where the sigmoid rounds to 1 (z > 17 in 32-bit)
    const float c = (!softmax && !correction && G == 1) ? z : s + (correction ? kf_load(correction, e) : 0.f);
    choice[e] = c == c ? c : NEG;                      // a row of padding may hold anything
  }
  __syncwarp();
  if (G > 1) {
    const int per = E / G;
    for (int g = lane; g < G; g += 32) {
      float a = NEG, b = NEG;                          // the two largest of the group
      for (int i = 0; i < per; ++i) {
        const float c = choice[g * per + i];
        if (c > a) { b = a; a = c; } else if (c > b) b = c;
      }
      gscore[g] = (per > 1 && group_best != 1) ? a + b : a;
    }
    __syncwarp();
    // the best `keep` groups stay; mark them by +inf one after the other, then close the others
    for (int r = 0; r < keep; ++r) {
      float best = NEG; int arg = -1;
      for (int g = lane; g < G; g += 32) {
        const float v = gscore[g];
        if (v != INFINITY && (arg < 0 || v > best)) { best = v; arg = g; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
        if (oa >= 0 && (arg < 0 || ob > best || (ob == best && oa < arg))) { best = ob; arg = oa; }
      }
      if (lane == 0 && arg >= 0) gscore[arg] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (gscore[e / per] != INFINITY) choice[e] = NEG;
    __syncwarp();
  }
  float sum = 0.f;
  for (int r = 0; r < top; ++r) {
    float best = NEG; int arg = -1;
    for (int e = lane; e < E; e += 32) {
      const float v = choice[e];
      if (v != INFINITY && (arg < 0 || v > best)) { best = v; arg = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (oa >= 0 && (arg < 0 || ob > best || (ob == best && oa < arg))) { best = ob; arg = oa; }
    }
    // arg is always a valid expert that was not taken yet (taken ones are marked +inf), also in a row of padding
    if (lane == 0) {
      ids[(size_t)t * top + r] = arg;
      choice[arg] = INFINITY;
    }
    __syncwarp();
    sum += score[arg];
  }
  for (int r = lane; r < top; r += 32) {
    const int e = ids[(size_t)t * top + r];
    weights[(size_t)t * top + r] = (normalize ? score[e] / (sum + 1e-20f) : score[e]) * scale;
  }
}

KF_API int kf_moe_route(const float* logits, const void* correction, int w_dtype, int T, int E, int G, int keep, int top,
                        float scale, int softmax, int group_best, int normalize, int* ids, float* weights, cudaStream_t stream) {
  if (T <= 0) return KF_OK;
  if (E < 1 || E > KF_MOE_MAX_EXPERTS || top < 1 || top > E || G < 1 || E % G || keep < 1 || keep > G) return KF_ERR_SIZE;
  if (G > 1 && keep * (E / G) < top) return KF_ERR_SIZE;
  const size_t smem = (size_t)4 * (2 * E + G) * sizeof(float);
  const dim3 grid(kf_ceil_div(T, 4));
  if (w_dtype == KF_F32)
    kf_launch(moe_route_kernel<float>, grid, dim3(128), smem, stream, logits, (const float*)correction, T, E, G, keep, top, scale, softmax, group_best, normalize, ids, weights);
  else if (w_dtype == KF_BF16)
    kf_launch(moe_route_kernel<__nv_bfloat16>, grid, dim3(128), smem, stream, logits, (const __nv_bfloat16*)correction, T, E, G, keep,
              top, scale, softmax, group_best, normalize, ids, weights);
  else return KF_ERR_DTYPE;
  KF_CHECK_LAUNCH();
  return KF_OK;
}

__global__ void __launch_bounds__(1024) moe_plan_kernel(const int* __restrict__ ids, int P, int E, int* __restrict__ sorted_pair,
                                                        int* __restrict__ inverse, int* __restrict__ tile_group,
                                                        int* __restrict__ tile_row0, int* __restrict__ tile_nrows,
                                                        int* __restrict__ n_tiles) {
  kf_pdl_trigger();
  kf_pdl_wait();
  __shared__ int cnt[KF_MOE_MAX_EXPERTS], off[KF_MOE_MAX_EXPERTS + 1], toff[KF_MOE_MAX_EXPERTS + 1];
  const int tid = threadIdx.x;
  for (int e = tid; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int i = tid; i < P; i += blockDim.x) atomicAdd(&cnt[ids[i]], 1);
  __syncthreads();
  if (tid == 0) {
    int a = 0, b = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = a; toff[e] = b;
      a += cnt[e];
      b += (cnt[e] + GM - 1) / GM;
    }
    off[E] = a; toff[E] = b;
    *n_tiles = b;
  }
  __syncthreads();
  for (int e = tid; e < E; e += blockDim.x) {
    const int n = cnt[e];
    for (int j = 0; j * GM < n; ++j) {
      tile_group[toff[e] + j] = e;
      tile_row0[toff[e] + j] = off[e] + j * GM;
      tile_nrows[toff[e] + j] = min(GM, n - j * GM);
    }
  }
  __syncthreads();
  for (int e = tid; e < E; e += blockDim.x) cnt[e] = 0;      // now the cursor of every expert
  __syncthreads();
  for (int i = tid; i < P; i += blockDim.x) {
    const int e = ids[i];
    const int pos = off[e] + atomicAdd(&cnt[e], 1);
    sorted_pair[pos] = i;
    inverse[i] = pos;
  }
}

// tile arrays hold P / 64 + E entries at most.
KF_API int kf_moe_plan(const int* ids, int P, int E, int* sorted_pair, int* inverse, int* tile_group, int* tile_row0,
                       int* tile_nrows, int* n_tiles, cudaStream_t stream) {
  if (P <= 0) return KF_OK;
  if (E < 1 || E > KF_MOE_MAX_EXPERTS) return KF_ERR_SIZE;
  kf_launch(moe_plan_kernel, dim3(1), dim3(1024), 0, stream, ids, P, E, sorted_pair, inverse, tile_group, tile_row0, tile_nrows, n_tiles);
  KF_CHECK_LAUNCH();
  return KF_OK;
}

__global__ void moe_combine_kernel(const float* __restrict__ expert_out, const int* __restrict__ inverse,
                                   const float* __restrict__ weights, const float* __restrict__ shared, float* __restrict__ y,
                                   int T, int W, int top) {
  kf_pdl_trigger();
  kf_pdl_wait();
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < top; ++j)
      acc = fmaf(weights ? weights[(size_t)t * top + j] : 1.f, expert_out[(size_t)inverse[(size_t)t * top + j] * W + i], acc);
    if (shared) acc += shared[(size_t)t * W + i];
    y[(size_t)t * W + i] = acc;
  }
}

KF_API int kf_moe_combine(const float* expert_out, const int* inverse, const float* weights, const float* shared, float* y,
                          int T, int W, int top, cudaStream_t stream) {
  if (T <= 0) return KF_OK;
  kf_launch(moe_combine_kernel, dim3(T), dim3(W >= 1024 ? 256 : 128), 0, stream, expert_out, inverse, weights, shared, y, T, W, top);
  KF_CHECK_LAUNCH();
  return KF_OK;
}
