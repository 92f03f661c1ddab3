// A matrix memory with exponential gates (the mLSTM cell): per head a d x dv state S, a d-vector n and a running
// maximum m of the gates' logarithms, all 32-bit, carried per request in state slots.
//
// For a token with raw gate values zi, zf of a head (columns of a 32-bit projection, plus a bias each):
//   gi = cap tanh(zi / cap)                       log input gate
//   gf = logsigmoid(cap tanh(zf / cap))           log forget gate
//   m' = max(gf + m, gi);   keep = exp(gf + m - m'),  take = exp(gi - m'),  floor = exp(-m')
//   S' = keep S + take k v^T;   n' = keep n + take k;   o = S'^T q / (max(|n' . q|, floor) + 1e-6),   q times d^-1/2
// m starts at 0 (a zeroed state slot), S and n at zero.
// State per (slot, head): S [d, dv]; and a row of ceil(dv / 16) copies of n (d numbers each) followed by m and three unused
// numbers.  Every block of the walk owns 16 value columns and ITS OWN copy of n, which it reads at its start and writes at
// its end: blocks of one head run at different times, and a shared n would be read by a late block after an early one had
// already moved it on.
//
// kf_mlstm_gates: one warp per (request, head) walks the request's rows 32 at a time.  Inside a chunk the maxima follow
//   from two scans: with F_j the running sum of gf, m_j = F_j + max(m_before, max_{s <= j}(gi_s - F_s)).  Any rounding of
//   m is harmless as long as keep, take and floor use the same values (they only move the stabiliser, and S, n and the
//   floor move with it); it writes (keep, take, floor, m) per (row, head) and, when the state is written, the last m.
// kf_mlstm_scan: the walk.  A block owns (request, head, 16 value columns); LANES = 4..32 lanes share a column (d / 8 of
//   them, so a block has 64 to 512 threads), each with eight rows of S and of n in registers: rows (g LANES + lane) 4 + i
//   for g = 0, 1 and i = 0..3, so that the lanes of a column read consecutive 16-byte pieces of q and k from shared
//   memory; q, k, v and the gates of 16 rows at a time are staged in shared memory,
//   in a ring of two stages filled by asynchronous 16-byte copies while the stage before is walked (plain loads when
//   sizes or addresses do not allow 16-byte copies).  Tokens are walked strictly in order with the same arithmetic whatever the portion, so a token's result does not
//   depend on how the prompt was cut.
#include "common.cuh"

constexpr int ML_R = 8;                // rows of the state a thread holds: two groups of four
constexpr int ML_COLS = 16;            // value columns per block
constexpr int ML_CHUNK = 16;           // rows staged at a time

__device__ __forceinline__ float ml_logsigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

template <typename TW>
__global__ void __launch_bounds__(128) mlstm_gates_kernel(const float* __restrict__ proj, int ld, int i0, int f0,
                                                          const TW* __restrict__ bi, const TW* __restrict__ bf, float cap,
                                                          float* __restrict__ nstate, int nstride, int m_at,
                                                          float* __restrict__ gates, int H, int n_reqs,
                                                          const int* __restrict__ req_row_start,
                                                          const int* __restrict__ req_n_rows,
                                                          const int* __restrict__ req_state_slot, int writes) {
  kf_pdl_trigger();
  kf_pdl_wait();
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= n_reqs * H) return;
  const int r = item / H, h = item - r * H;
  const int n = req_n_rows[r], row0 = req_row_start[r], slot = req_state_slot[r];
  if (n <= 0 || slot < 0) return;
  float* mp = nstate + ((size_t)slot * H + h) * nstride + m_at;
  float m_before = *mp;
  const float b_i = bi ? kf_load(bi, h) : 0.f, b_f = bf ? kf_load(bf, h) : 0.f;
  for (int c0 = 0; c0 < n; c0 += 32) {
    const int j = c0 + lane;
    const bool valid = j < n;
    float gi = -INFINITY, gf = 0.f;
    if (valid) {
      const float* src = proj + (size_t)(row0 + j) * ld;
      gi = cap * tanhf((src[i0 + h] + b_i) / cap);
      gf = ml_logsigmoid(cap * tanhf((src[f0 + h] + b_f) / cap));
    }
    float F = gf;                                            // inclusive running sum of gf over the chunk
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float u = __shfl_up_sync(0xffffffffu, F, o);
      if (lane >= o) F += u;
    }
    float g = gi - F;                                        // inclusive running maximum of gi_s - F_s
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float u = __shfl_up_sync(0xffffffffu, g, o);
      if (lane >= o) g = fmaxf(g, u);
    }
    const float m = F + fmaxf(m_before, g);
    float m_prev = __shfl_up_sync(0xffffffffu, m, 1);
    if (lane == 0) m_prev = m_before;
    if (valid) {
      float4 out;
      out.x = expf(gf + m_prev - m);
      out.y = expf(gi - m);
      out.z = expf(-m);
      out.w = m;
      reinterpret_cast<float4*>(gates)[(size_t)(row0 + j) * H + h] = out;
    }
    m_before = __shfl_sync(0xffffffffu, m, 31);              // lanes beyond the last row carry it on unchanged
  }
  if (writes && lane == 0) *mp = m_before;
}

KF_API int kf_mlstm_gates(const float* proj, int ld, int i0, int f0, const void* bi, const void* bf, int w_dtype, float cap,
                          float* nstate, int nstride, int m_at, float* gates, int H, int n_reqs, const int* req_row_start,
                          const int* req_n_rows, const int* req_state_slot, int writes, cudaStream_t stream) {
  if (n_reqs <= 0 || H <= 0) return KF_OK;
  if (!(cap > 0.f)) return KF_ERR_SIZE;
  const dim3 grid(kf_ceil_div((long)n_reqs * H, 4));
#define KF_GO(TW)                                                                                                     \
  kf_launch(mlstm_gates_kernel<TW>, grid, dim3(128), 0, stream, proj, ld, i0, f0, (const TW*)bi, (const TW*)bf, cap, nstate, \
            nstride, m_at, gates, H, n_reqs, req_row_start, req_n_rows, req_state_slot, writes)
  if (w_dtype == KF_F32) KF_GO(float);
  else if (w_dtype == KF_BF16) KF_GO(__nv_bfloat16);
  else return KF_ERR_DTYPE;
#undef KF_GO
  KF_CHECK_LAUNCH();
  return KF_OK;
}

struct KfMlstmArgs {
  const float* proj; int ld, q0, k0, v0;       // 32-bit rows: q (H d), k (H d), v (H dv) column ranges
  const float* gates;                          // [rows, H] of (keep, take, floor, m)
  float* S; float* nstate; int nstride;        // [slots, H, d, dv]; [slots, H, nstride]: a copy of n per block of 16 columns
  float* out;                                  // [rows, H dv]
  int H, d, dv, n_reqs;
  float q_scale;
  const int* req_row_start; const int* req_n_rows; const int* req_state_slot;
  int writes;
};

__device__ __forceinline__ void ml_cp16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void ml_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void ml_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// VEC: rows, column ranges and the gates' records start on 16-byte boundaries and d, dv are multiples of four, so a
// stage is filled by asynchronous 16-byte copies while the stage before it is walked; otherwise by plain loads.
template <int LANES, bool VEC>
__global__ void __launch_bounds__(LANES * ML_COLS) mlstm_scan_kernel(KfMlstmArgs p) {
  kf_pdl_trigger();
  kf_pdl_wait();
  extern __shared__ __align__(16) float sm[];
  constexpr int R = ML_R, THREADS = LANES * ML_COLS;
  constexpr int DP = R * LANES;                              // rows of the state a block holds (>= d, tails zero)
  constexpr int STAGE = 2 * ML_CHUNK * DP + ML_CHUNK * ML_COLS + ML_CHUNK * 4;
  const int col_blocks = (p.dv + ML_COLS - 1) / ML_COLS;
  const int cb = blockIdx.x % col_blocks;
  const int rh = blockIdx.x / col_blocks;
  const int h = rh % p.H, r = rh / p.H;
  const int n = p.req_n_rows[r], row0 = p.req_row_start[r], slot = p.req_state_slot[r];
  if (n <= 0 || slot < 0) return;
  const int tid = threadIdx.x, l = tid % LANES, cl = tid / LANES;
  const int col = cb * ML_COLS + cl;
  const bool live = col < p.dv;
  const int d = p.d, dv = p.dv;
  float S[R], nn[R];
  float* Sg = p.S + ((size_t)slot * p.H + h) * d * dv;
  float* ng = p.nstate + ((size_t)slot * p.H + h) * p.nstride + (size_t)cb * d;      // this block's own copy of n
  auto row_of = [&](int k) { return ((k >> 2) * LANES + l) * 4 + (k & 3); };
#pragma unroll
  for (int k = 0; k < R; ++k) {
    const int row = row_of(k);
    S[k] = (live && row < d) ? Sg[(size_t)row * dv + col] : 0.f;
    nn[k] = row < d ? ng[row] : 0.f;
  }
  // a stage: q [ML_CHUNK][DP], k [ML_CHUNK][DP], v [ML_CHUNK][ML_COLS], gates [ML_CHUNK][4]
  auto fill = [&](int c0, int st) {
    float* qs = sm + st * STAGE;
    float* ks = qs + ML_CHUNK * DP;
    float* vs = ks + ML_CHUNK * DP;
    float* gs = vs + ML_CHUNK * ML_COLS;
    const int rows = min(ML_CHUNK, n - c0);
    if constexpr (VEC) {
      for (int i = tid; i < rows * (DP / 4); i += THREADS) {
        const int t = i / (DP / 4), e = (i - t * (DP / 4)) * 4;
        const float* src = p.proj + (size_t)(row0 + c0 + t) * p.ld + h * d + e;
        if (e < d) { ml_cp16(qs + t * DP + e, src + p.q0); ml_cp16(ks + t * DP + e, src + p.k0); }
        else {
          *reinterpret_cast<float4*>(qs + t * DP + e) = make_float4(0.f, 0.f, 0.f, 0.f);
          *reinterpret_cast<float4*>(ks + t * DP + e) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
      for (int i = tid; i < rows * (ML_COLS / 4); i += THREADS) {
        const int t = i / (ML_COLS / 4), e = (i - t * (ML_COLS / 4)) * 4;
        const int c = cb * ML_COLS + e;
        if (c < dv) ml_cp16(vs + t * ML_COLS + e, p.proj + (size_t)(row0 + c0 + t) * p.ld + p.v0 + h * dv + c);
        else *reinterpret_cast<float4*>(vs + t * ML_COLS + e) = make_float4(0.f, 0.f, 0.f, 0.f);
      }
      for (int t = tid; t < rows; t += THREADS) ml_cp16(gs + t * 4, p.gates + ((size_t)(row0 + c0 + t) * p.H + h) * 4);
    } else {
      for (int i = tid; i < rows * DP; i += THREADS) {
        const int t = i / DP, e = i - t * DP;
        const float* src = p.proj + (size_t)(row0 + c0 + t) * p.ld;
        qs[i] = e < d ? src[p.q0 + h * d + e] : 0.f;
        ks[i] = e < d ? src[p.k0 + h * d + e] : 0.f;
      }
      for (int i = tid; i < rows * ML_COLS; i += THREADS) {
        const int t = i / ML_COLS, e = i - t * ML_COLS;
        const int c = cb * ML_COLS + e;
        vs[i] = c < dv ? p.proj[(size_t)(row0 + c0 + t) * p.ld + p.v0 + h * dv + c] : 0.f;
      }
      for (int i = tid; i < rows * 4; i += THREADS)
        gs[i] = p.gates[((size_t)(row0 + c0 + (i >> 2)) * p.H + h) * 4 + (i & 3)];
    }
  };
  fill(0, 0);
  ml_commit();
  int st = 0;
  for (int c0 = 0; c0 < n; c0 += ML_CHUNK, st ^= 1) {
    const int rows = min(ML_CHUNK, n - c0);
    if (c0 + ML_CHUNK < n) fill(c0 + ML_CHUNK, st ^ 1);      // the next rows arrive while these are walked
    ml_commit();
    ml_wait<1>();
    __syncthreads();
    const float* qs = sm + st * STAGE;
    const float* ks = qs + ML_CHUNK * DP;
    const float* vs = ks + ML_CHUNK * DP;
    const float* gs = vs + ML_CHUNK * ML_COLS;
    for (int t = 0; t < rows; ++t) {
      const float4 gt = *reinterpret_cast<const float4*>(gs + t * 4);          // keep, take, floor, m
      const float keep = gt.x, take = gt.y;
      const float tv = take * vs[t * ML_COLS + cl];
      float acc[4] = {0.f, 0.f, 0.f, 0.f}, nq[4] = {0.f, 0.f, 0.f, 0.f};       // four chains each, summed in a fixed order
#pragma unroll
      for (int g = 0; g < R / 4; ++g) {
        const int j = g * 4;
        const float4 kk = *reinterpret_cast<const float4*>(ks + t * DP + (g * LANES + l) * 4);
        const float4 qq = *reinterpret_cast<const float4*>(qs + t * DP + (g * LANES + l) * 4);
        S[j] = fmaf(keep, S[j], kk.x * tv);         nn[j] = fmaf(keep, nn[j], take * kk.x);
        S[j + 1] = fmaf(keep, S[j + 1], kk.y * tv); nn[j + 1] = fmaf(keep, nn[j + 1], take * kk.y);
        S[j + 2] = fmaf(keep, S[j + 2], kk.z * tv); nn[j + 2] = fmaf(keep, nn[j + 2], take * kk.z);
        S[j + 3] = fmaf(keep, S[j + 3], kk.w * tv); nn[j + 3] = fmaf(keep, nn[j + 3], take * kk.w);
        acc[0] = fmaf(S[j], qq.x, acc[0]);     nq[0] = fmaf(nn[j], qq.x, nq[0]);
        acc[1] = fmaf(S[j + 1], qq.y, acc[1]); nq[1] = fmaf(nn[j + 1], qq.y, nq[1]);
        acc[2] = fmaf(S[j + 2], qq.z, acc[2]); nq[2] = fmaf(nn[j + 2], qq.z, nq[2]);
        acc[3] = fmaf(S[j + 3], qq.w, acc[3]); nq[3] = fmaf(nn[j + 3], qq.w, nq[3]);
      }
      float a = (acc[0] + acc[1]) + (acc[2] + acc[3]), b = (nq[0] + nq[1]) + (nq[2] + nq[3]);
#pragma unroll
      for (int o = LANES / 2; o > 0; o >>= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, o);
        b += __shfl_xor_sync(0xffffffffu, b, o);
      }
      if (l == 0 && live)                                     // q times d^-1/2 multiplies both sums
        p.out[(size_t)(row0 + c0 + t) * p.H * dv + h * dv + col] =
            __fdividef(a * p.q_scale, fmaxf(fabsf(b * p.q_scale), gt.z) + 1e-6f);
    }
    __syncthreads();                                         // this stage is filled again in the next turn
  }
  ml_wait<0>();
  if (!p.writes) return;
#pragma unroll
  for (int k = 0; k < R; ++k) {
    const int row = row_of(k);
    if (live && row < d) Sg[(size_t)row * dv + col] = S[k];
    if (cl == 0 && row < d) ng[row] = nn[k];
  }
}

KF_API int kf_mlstm_scan(const float* proj, int ld, int q0, int k0, int v0, const float* gates, float* S, float* nstate,
                         int nstride, float* out, int H, int d, int dv, float q_scale, int n_reqs, const int* req_row_start,
                         const int* req_n_rows, const int* req_state_slot, int writes, cudaStream_t stream) {
  if (n_reqs <= 0) return KF_OK;
  if (d < 1 || d > 256 || dv < 1 || H < 1 || nstride < ((dv + ML_COLS - 1) / ML_COLS) * d) return KF_ERR_SIZE;
  KfMlstmArgs p{proj, ld, q0, k0, v0, gates, S, nstate, nstride, out, H, d, dv, n_reqs, q_scale, req_row_start, req_n_rows,
                req_state_slot, writes};
  const int col_blocks = (dv + ML_COLS - 1) / ML_COLS;
  const dim3 grid((unsigned)((long)n_reqs * H * col_blocks));
  const int lanes = d <= 32 ? 4 : (d <= 64 ? 8 : (d <= 128 ? 16 : 32));
  const size_t smem = 2 * (size_t)(2 * ML_CHUNK * ML_R * lanes + ML_CHUNK * ML_COLS + ML_CHUNK * 4) * sizeof(float);
  const bool vec = d % 4 == 0 && dv % 4 == 0 && ld % 4 == 0 && q0 % 4 == 0 && k0 % 4 == 0 && v0 % 4 == 0 &&
                   (((uintptr_t)proj | (uintptr_t)gates) & 15) == 0;
#define KF_GO(LL)                                                                                               \
  do {                                                                                                          \
    if (vec) {                                                                                                  \
      if (smem > 48 * 1024) cudaFuncSetAttribute(mlstm_scan_kernel<LL, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      kf_launch(mlstm_scan_kernel<LL, true>, grid, dim3(LL * ML_COLS), smem, stream, p);                         \
    } else {                                                                                                    \
      if (smem > 48 * 1024) cudaFuncSetAttribute(mlstm_scan_kernel<LL, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      kf_launch(mlstm_scan_kernel<LL, false>, grid, dim3(LL * ML_COLS), smem, stream, p);                        \
    }                                                                                                           \
  } while (0)
  if (lanes == 4) KF_GO(4);
  else if (lanes == 8) KF_GO(8);
  else if (lanes == 16) KF_GO(16);
  else KF_GO(32);
#undef KF_GO
  KF_CHECK_LAUNCH();
  return KF_OK;
}
