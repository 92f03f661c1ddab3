// A matrix memory with exponential gates (the mLSTM cell): per head a d x dv state S, a d-vector n and a running
// maximum m of the gates' logarithms, all 32-bit, carried per request in state slots.
//
// For a token with raw gate values zi, zf of a head (columns of a 32-bit projection, plus a bias each):
//   gi = cap tanh(zi / cap)                       log input gate
//   gf = logsigmoid(cap tanh(zf / cap))           log forget gate
//   m' = max(gf + m, gi);   keep = exp(gf + m - m'),  take = exp(gi - m'),  floor = exp(-m')
//   S' = keep S + take k v^T;   n' = keep n + take k;   o = S'^T q / (max(|n' . q|, floor) + 1e-6),   q times d^-1/2
// m starts at 0 (a zeroed state slot), S and n at zero.
//
// kf_mlstm_gates: one warp per (request, head) walks the request's rows 32 at a time.  Inside a chunk the maxima follow
//   from two scans: with F_j the running sum of gf, m_j = F_j + max(m_before, max_{s <= j}(gi_s - F_s)).  Any rounding of
//   m is harmless as long as keep, take and floor use the same values (they only move the stabiliser, and S, n and the
//   floor move with it); it writes (keep, take, floor, m) per (row, head) and, when the state is written, the last m.
// kf_mlstm_scan: the walk.  A block owns (request, head, 16 value columns); eight lanes share a column, each with R
//   consecutive rows of S and of n in registers; q, k, v and the gates of 16 rows at a time are staged in shared memory.
//   Tokens are walked strictly in order with the same arithmetic whatever the portion, so a token's result does not
//   depend on how the prompt was cut.
#include "common.cuh"

constexpr int ML_LANES = 8;            // lanes that share a value column
constexpr int ML_COLS = 16;            // value columns per block
constexpr int ML_THREADS = ML_LANES * ML_COLS;
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
  float* S; float* nstate; int nstride;        // [slots, H, d, dv]; [slots, H, nstride] with n in the first d places
  float* out;                                  // [rows, H dv]
  int H, d, dv, n_reqs;
  float q_scale;
  const int* req_row_start; const int* req_n_rows; const int* req_state_slot;
  int writes;
};

template <int R>
__global__ void __launch_bounds__(ML_THREADS) mlstm_scan_kernel(KfMlstmArgs p) {
  kf_pdl_trigger();
  kf_pdl_wait();
  extern __shared__ float sm[];
  const int DP = R * ML_LANES;                               // rows of the state a block holds (>= d, tails zero)
  float* qs = sm;                                            // [ML_CHUNK][DP]
  float* ks = qs + ML_CHUNK * DP;                            // [ML_CHUNK][DP]
  float* vs = ks + ML_CHUNK * DP;                            // [ML_CHUNK][ML_COLS]
  float* gs = vs + ML_CHUNK * ML_COLS;                       // [ML_CHUNK][4]
  const int col_blocks = (p.dv + ML_COLS - 1) / ML_COLS;
  const int cb = blockIdx.x % col_blocks;
  const int rh = blockIdx.x / col_blocks;
  const int h = rh % p.H, r = rh / p.H;
  const int n = p.req_n_rows[r], row0 = p.req_row_start[r], slot = p.req_state_slot[r];
  if (n <= 0 || slot < 0) return;
  const int tid = threadIdx.x, l = tid % ML_LANES, cl = tid / ML_LANES;
  const int col = cb * ML_COLS + cl;
  const bool live = col < p.dv;
  const int d = p.d, dv = p.dv;
  float S[R], nn[R];
  float* Sg = p.S + ((size_t)slot * p.H + h) * d * dv;
  float* ng = p.nstate + ((size_t)slot * p.H + h) * p.nstride;
#pragma unroll
  for (int k = 0; k < R; ++k) {
    const int row = l * R + k;
    S[k] = (live && row < d) ? Sg[(size_t)row * dv + col] : 0.f;
    nn[k] = row < d ? ng[row] : 0.f;
  }
  for (int c0 = 0; c0 < n; c0 += ML_CHUNK) {
    const int rows = min(ML_CHUNK, n - c0);
    __syncthreads();                                         // the chunk before has been walked
    for (int i = tid; i < rows * DP; i += ML_THREADS) {
      const int t = i / DP, e = i - t * DP;
      const float* src = p.proj + (size_t)(row0 + c0 + t) * p.ld;
      qs[i] = e < d ? src[p.q0 + h * d + e] * p.q_scale : 0.f;
      ks[i] = e < d ? src[p.k0 + h * d + e] : 0.f;
    }
    for (int i = tid; i < rows * ML_COLS; i += ML_THREADS) {
      const int t = i / ML_COLS, e = i - t * ML_COLS;
      const int c = cb * ML_COLS + e;
      vs[i] = c < dv ? p.proj[(size_t)(row0 + c0 + t) * p.ld + p.v0 + h * dv + c] : 0.f;
    }
    for (int i = tid; i < rows * 4; i += ML_THREADS)
      gs[i] = p.gates[((size_t)(row0 + c0 + (i >> 2)) * p.H + h) * 4 + (i & 3)];
    __syncthreads();
    for (int t = 0; t < rows; ++t) {
      const float keep = gs[t * 4], take = gs[t * 4 + 1], floor_ = gs[t * 4 + 2];
      const float tv = take * vs[t * ML_COLS + cl];
      const float* q = qs + t * DP + l * R;
      const float* k = ks + t * DP + l * R;
      float acc = 0.f, nq = 0.f;
#pragma unroll
      for (int j = 0; j < R; ++j) {
        S[j] = fmaf(keep, S[j], k[j] * tv);
        nn[j] = fmaf(keep, nn[j], take * k[j]);
        acc = fmaf(S[j], q[j], acc);
        nq = fmaf(nn[j], q[j], nq);
      }
#pragma unroll
      for (int o = ML_LANES / 2; o > 0; o >>= 1) {
        acc += __shfl_xor_sync(0xffffffffu, acc, o);
        nq += __shfl_xor_sync(0xffffffffu, nq, o);
      }
      if (l == 0 && live)
        p.out[(size_t)(row0 + c0 + t) * p.H * dv + h * dv + col] = acc / (fmaxf(fabsf(nq), floor_) + 1e-6f);
    }
  }
  if (!p.writes) return;
#pragma unroll
  for (int k = 0; k < R; ++k) {
    const int row = l * R + k;
    if (live && row < d) Sg[(size_t)row * dv + col] = S[k];
    if (cb == 0 && cl == 0 && row < d) ng[row] = nn[k];
  }
}

KF_API int kf_mlstm_scan(const float* proj, int ld, int q0, int k0, int v0, const float* gates, float* S, float* nstate,
                         int nstride, float* out, int H, int d, int dv, float q_scale, int n_reqs, const int* req_row_start,
                         const int* req_n_rows, const int* req_state_slot, int writes, cudaStream_t stream) {
  if (n_reqs <= 0) return KF_OK;
  if (d < 1 || d > 256 || dv < 1 || H < 1 || nstride < d) return KF_ERR_SIZE;
  KfMlstmArgs p{proj, ld, q0, k0, v0, gates, S, nstate, nstride, out, H, d, dv, n_reqs, q_scale, req_row_start, req_n_rows,
                req_state_slot, writes};
  const int col_blocks = (dv + ML_COLS - 1) / ML_COLS;
  const dim3 grid((unsigned)((long)n_reqs * H * col_blocks));
  const int R = d <= 32 ? 4 : (d <= 64 ? 8 : (d <= 128 ? 16 : 32));
  const size_t smem = (size_t)(2 * ML_CHUNK * R * ML_LANES + ML_CHUNK * ML_COLS + ML_CHUNK * 4) * sizeof(float);
#define KF_GO(RR) kf_launch(mlstm_scan_kernel<RR>, grid, dim3(ML_THREADS), smem, stream, p)
  if (R == 4) KF_GO(4);
  else if (R == 8) KF_GO(8);
  else if (R == 16) KF_GO(16);
  else KF_GO(32);
#undef KF_GO
  KF_CHECK_LAUNCH();
  return KF_OK;
}
