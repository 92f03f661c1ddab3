// The gated delta rule: a recurrent mixer whose state per head is a d x dv matrix S of 32-bit floats (rows = key
// channels, columns = value channels) that is decayed, corrected towards the current value and read, token by token:
//   S <- diag(g_t) S          g_t: one decay per head, or one per head and key channel (rows of S)
//   u  = beta_t (v_t - S^T k_t)
//   S <- S + k_t u^T
//   o_t = S^T q_t             (the read-out sees the current token's write)
// with q, k unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q also times d^(-1/2), beta = sigmoid(raw),
// g = exp(-exp(A_log_h) * softplus(raw + dt_bias)).  Query/key head of value head h: h / (heads / kv_heads).
// Everything here is 32-bit.  The tokens of a request are walked in order with the same arithmetic whatever the step
// holds of it (one token, a portion, a whole prompt), and the state is carried exactly: a token's result does not depend
// on how the sequence was cut.
//
// Two kernels.  What does not depend on the state (the unit vectors, the sigmoid, the decays: the transcendental work)
// is computed once per (row, head), side by side over the whole step, and left laid out as the walk stages it.
// The walk: a block of 128 threads owns (request, head, 128 / LANES value columns).  Thread (c, l) keeps rows
// l*NR .. l*NR+NR-1 of column c in registers (d <= LANES * NR; rows beyond d are zero and stay zero); the LANES lanes of
// a column add their shares of S^T k by shuffles (the one reduction on the chain from token to token), each from four
// interleaved partial sums held as two pairs that packed instructions (fma.rn.f32x2) update, as they update pairs of
// neighbouring rows of S; their shares of S^T q go to shared
// memory and are summed, in a fixed order, after the walk over the stage.  Rows of R tokens at a time arrive in shared
// memory by 16-byte cp.async copies into one of two stages while the stage before is walked, so that the serial walk is
// multiply-adds and shared loads only.  A lane's chunk of a staged row starts every LS floats (NR + 4; NR where that is
// 4): the lanes of a column then read different banks with 16-byte loads.  With one long prompt in a step the walk
// has heads x d x dv / NR threads and no more, so NR is small: what limits it is the latency of a warp's chain, which
// only more warps per scheduler hide.
//
// kf_head_norm_gate follows: every head's o is divided by its root mean square over dv, times a weight vector shared
// by the heads (w_stride 0) or one per head (w_stride dv: head h reads w[h * dv ..]), times silu or sigmoid of a gate column.
#include "common.cuh"

struct KfDeltaArgs {
  const float* qkv; int ld_qkv, q0, k0, v0;      // 32-bit rows after the short convolution and its activation
  const float* beta; int ld_beta, beta0;         // raw beta of head h: column beta0 + h
  const float* decay; int ld_decay, decay0;      // raw decay: column decay0 + h, or decay0 + h * d + i per key channel
  int per_channel;
  const void* dt_bias; const void* a_log;        // [H] or [H * d]; [H]
  float* state;                                  // [slots, H, d, dv]
  float* out; int ld_out;                        // [rows, H * dv]
  int H, KH, d, dv, n_reqs;
  const int* req_row_start; const int* req_n_rows; const int* req_state_slot;
  int writes;
};

__device__ __forceinline__ float kf_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

__device__ __forceinline__ void kf_cp_async4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void kf_cp_async16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// Everything of a token that does not depend on the state, once per (row, head) and side by side over the whole step:
// the unit vectors q (times d^-1/2) and k, the decays (per key channel, or one) and beta.  q, k and the decays are
// written as the walk wants them in shared memory (a lane's chunk of NR numbers every LS floats; any floats
// between chunks are never read), so that a stage of the walk is filled by 16-byte copies:
//   prep[((row * H + h) * 3 + {0: q, 1: k, 2: decays}) * ROW + (i / NR) * LS + i % NR],   small[(row * H + h) * 2 + {0: beta, 1: decay}]
template <typename TW>
__global__ void __launch_bounds__(128) delta_prepare_kernel(KfDeltaArgs p, float* __restrict__ prep, float* __restrict__ small,
                                                            int T, int NR, int LANES) {
  kf_pdl_trigger();
  kf_pdl_wait();
  const int lane = threadIdx.x & 31;
  const long item = (long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= (long)T * p.H) return;
  const int t = (int)(item / p.H), h = (int)(item - (long)t * p.H);
  const int kh = h / (p.H / p.KH), d = p.d, LS = NR == 4 ? 4 : NR + 4, ROW = LANES * LS, DP = NR * LANES;
  const float* qs = p.qkv + (size_t)t * p.ld_qkv + p.q0 + kh * d;
  const float* ks = p.qkv + (size_t)t * p.ld_qkv + p.k0 + kh * d;
  float sq = 0.f, sk = 0.f;
  for (int i = lane; i < d; i += 32) {
    sq = fmaf(qs[i], qs[i], sq);
    sk = fmaf(ks[i], ks[i], sk);
  }
  sq = kf_warp_sum(sq);
  sk = kf_warp_sum(sk);
  const float fq = 1.f / sqrtf((float)d) / sqrtf(sq + 1e-6f), fk = 1.f / sqrtf(sk + 1e-6f);
  const float rate = expf(kf_load((const TW*)p.a_log, h));
  float* dst = prep + (size_t)item * 3 * ROW;
  for (int i = lane; i < DP; i += 32) {
    const int at = (i / NR) * LS + (i % NR);
    const bool in = i < d;
    dst[at] = in ? qs[i] * fq : 0.f;
    dst[ROW + at] = in ? ks[i] * fk : 0.f;
    if (p.per_channel) {
      float g = 1.f;
      if (in) g = expf(-rate * kf_softplus(p.decay[(size_t)t * p.ld_decay + p.decay0 + h * d + i] + kf_load((const TW*)p.dt_bias, h * d + i)));
      dst[2 * ROW + at] = g;
    }
  }
  if (lane == 0) {
    small[item * 2] = 1.f / (1.f + expf(-p.beta[(size_t)t * p.ld_beta + p.beta0 + h]));
    if (!p.per_channel)
      small[item * 2 + 1] = expf(-rate * kf_softplus(p.decay[(size_t)t * p.ld_decay + p.decay0 + h] + kf_load((const TW*)p.dt_bias, h)));
  }
}

// The walk.  NR rows of a column per thread, LANES threads per column (d <= NR * LANES), THREADS / LANES columns per block.
template <int NR, int LANES, int THREADS>
__global__ void __launch_bounds__(THREADS) delta_rule_kernel(KfDeltaArgs p, const float* __restrict__ prep, const float* __restrict__ small) {
  kf_pdl_trigger();
  kf_pdl_wait();
  constexpr int CB = THREADS / LANES;            // value columns of a block
  constexpr int LS = NR == 4 ? 4 : NR + 4;       // floats between the chunks of two lanes (16-byte loads of the lanes of a
                                                 // quarter warp then fall into different banks)
  constexpr int ROW = LANES * LS;
  constexpr int R = ROW > 200 ? 4 : 8;           // tokens staged at a time
  __shared__ __align__(16) float q_s[2][R][ROW];
  __shared__ __align__(16) float k_s[2][R][ROW];
  __shared__ __align__(16) float g_s[2][R][ROW];
  __shared__ float v_s[2][R][CB];
  __shared__ float small_s[2][R][2];
  __shared__ float o_part[2][R][CB][LANES + 1];  // every lane's share of o: summed over the lanes after the walk
  const int req = blockIdx.x / p.H, h = blockIdx.x - req * p.H;
  const int n = p.req_n_rows[req];
  if (n <= 0) return;
  const int row0 = p.req_row_start[req], slot = p.req_state_slot[req];
  const int tid = threadIdx.x, c = tid / LANES, l = tid % LANES;
  const int col0 = blockIdx.y * CB, col = col0 + c;
  const bool col_ok = col < p.dv;
  const int d = p.d, dv = p.dv;
  float2 S[NR / 2];                              // rows l*NR + 2j and + 2j + 1: one packed instruction updates both
  float* sp = p.state + ((size_t)slot * p.H + h) * d * dv;
#pragma unroll
  for (int j = 0; j < NR / 2; ++j) {
    const int r = l * NR + 2 * j;
    S[j].x = (r < d && col_ok) ? sp[(size_t)r * dv + col] : 0.f;
    S[j].y = (r + 1 < d && col_ok) ? sp[(size_t)(r + 1) * dv + col] : 0.f;
  }

  // rows t0 .. t0 + nr - 1 of the request into stage `buf` (asynchronous copies, 16 bytes where the source allows)
  auto issue = [&](int buf, int t0, int nr) {
    constexpr int V4 = ROW / 4;
    for (int idx = tid; idx < nr * V4; idx += THREADS) {
      const int tt = idx / V4, j = idx - tt * V4;
      const float* src = prep + ((size_t)(row0 + t0 + tt) * p.H + h) * 3 * ROW + j * 4;
      kf_cp_async16(&q_s[buf][tt][j * 4], src);
      kf_cp_async16(&k_s[buf][tt][j * 4], src + ROW);
      if (p.per_channel) kf_cp_async16(&g_s[buf][tt][j * 4], src + 2 * ROW);
    }
    for (int idx = tid; idx < nr * CB; idx += THREADS) {
      const int tt = idx / CB, cc = idx - tt * CB;
      if (col0 + cc < dv) kf_cp_async4(&v_s[buf][tt][cc], p.qkv + (size_t)(row0 + t0 + tt) * p.ld_qkv + p.v0 + h * dv + col0 + cc);
      else v_s[buf][tt][cc] = 0.f;
    }
    if (tid < nr * 2) kf_cp_async4(&small_s[buf][tid >> 1][tid & 1], small + ((size_t)(row0 + t0 + (tid >> 1)) * p.H + h) * 2 + (tid & 1));
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // o of the rows t0 .. t0 + nr - 1, whose lanes' shares stand in o_part[buf]: lane sums in a fixed order, then the store
  auto finish = [&](int buf, int t0, int nr) {
    for (int idx = tid; idx < nr * CB; idx += THREADS) {
      const int tt = idx / CB, cc = idx - tt * CB;
      if (col0 + cc >= dv) continue;
      float o = 0.f;
#pragma unroll
      for (int j = 0; j < LANES; ++j) o += o_part[buf][tt][cc][j];
      p.out[(size_t)(row0 + t0 + tt) * p.ld_out + h * dv + col0 + cc] = o;
    }
  };

  const int n_chunks = (n + R - 1) / R;
  issue(0, 0, min(R, n));
  for (int ch = 0; ch < n_chunks; ++ch) {
    const int buf = ch & 1, t0 = ch * R, nr = min(R, n - t0);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                             // this stage has landed; the walk over the stage before is over
    if (ch + 1 < n_chunks) issue(buf ^ 1, t0 + R, min(R, n - t0 - R));
    if (ch > 0) finish(buf ^ 1, t0 - R, R);
#pragma unroll 2
    for (int tt = 0; tt < nr; ++tt) {              // the walk
      const float* kq = &k_s[buf][tt][l * LS];
      const float* qq = &q_s[buf][tt][l * LS];
      float2 kr[NR / 2];
      float2 kva = make_float2(0.f, 0.f), kvb = make_float2(0.f, 0.f);
      if (p.per_channel) {
        const float* gq = &g_s[buf][tt][l * LS];
#pragma unroll
        for (int i = 0; i < NR; i += 4) {
          const float4 g4 = *reinterpret_cast<const float4*>(gq + i);
          const float4 k4 = *reinterpret_cast<const float4*>(kq + i);
          kr[i / 2] = make_float2(k4.x, k4.y); kr[i / 2 + 1] = make_float2(k4.z, k4.w);
          S[i / 2] = __fmul2_rn(S[i / 2], make_float2(g4.x, g4.y));
          S[i / 2 + 1] = __fmul2_rn(S[i / 2 + 1], make_float2(g4.z, g4.w));
          kva = __ffma2_rn(S[i / 2], kr[i / 2], kva);
          kvb = __ffma2_rn(S[i / 2 + 1], kr[i / 2 + 1], kvb);
        }
      } else {
        const float g = small_s[buf][tt][1];
        const float2 g2 = make_float2(g, g);
#pragma unroll
        for (int i = 0; i < NR; i += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(kq + i);
          kr[i / 2] = make_float2(k4.x, k4.y); kr[i / 2 + 1] = make_float2(k4.z, k4.w);
          S[i / 2] = __fmul2_rn(S[i / 2], g2);
          S[i / 2 + 1] = __fmul2_rn(S[i / 2 + 1], g2);
          kva = __ffma2_rn(S[i / 2], kr[i / 2], kva);
          kvb = __ffma2_rn(S[i / 2 + 1], kr[i / 2 + 1], kvb);
        }
      }
      float kv = (kva.x + kva.y) + (kvb.x + kvb.y);
#pragma unroll
      for (int o = 1; o < LANES; o <<= 1) kv += __shfl_xor_sync(0xffffffffu, kv, o);
      const float u = small_s[buf][tt][0] * (v_s[buf][tt][c] - kv);
      const float2 u2 = make_float2(u, u);
      float2 oa = make_float2(0.f, 0.f), ob = make_float2(0.f, 0.f);
#pragma unroll
      for (int i = 0; i < NR; i += 4) {
        const float4 q4 = *reinterpret_cast<const float4*>(qq + i);
        S[i / 2] = __ffma2_rn(kr[i / 2], u2, S[i / 2]);
        S[i / 2 + 1] = __ffma2_rn(kr[i / 2 + 1], u2, S[i / 2 + 1]);
        oa = __ffma2_rn(S[i / 2], make_float2(q4.x, q4.y), oa);
        ob = __ffma2_rn(S[i / 2 + 1], make_float2(q4.z, q4.w), ob);
      }
      o_part[buf][tt][c][l] = (oa.x + oa.y) + (ob.x + ob.y);   // off the chain from token to token: summed by `finish`
    }
  }
  __syncthreads();
  finish((n_chunks - 1) & 1, (n_chunks - 1) * R, n - (n_chunks - 1) * R);
  if (p.writes) {
#pragma unroll
    for (int j = 0; j < NR / 2; ++j) {
      const int r = l * NR + 2 * j;
      if (r < d && col_ok) sp[(size_t)r * dv + col] = S[j].x;
      if (r + 1 < d && col_ok) sp[(size_t)(r + 1) * dv + col] = S[j].y;
    }
  }
}

// Rows per thread, lanes per column and threads per block by key size: few rows per thread, because one long prompt has
// heads x d x dv / NR threads and no more, and only several warps per scheduler hide the latency of a warp's chain.
static void delta_shape(int d, int* nr, int* lanes, int* threads) {
  // (measured at 16 heads x 128 x 128, one prompt of 2,048 tokens: 8 rows x 16 lanes 666 us; 4 rows x 32 lanes in blocks of
  // 256 threads 771 us, its fifth shuffle step costing more than the second warp per scheduler hides; 16 rows x 8 lanes 1,010 us)
  if (d <= 32) { *nr = 8; *lanes = 4; *threads = 128; }
  else if (d <= 64) { *nr = 8; *lanes = 8; *threads = 128; }
  else if (d <= 128) { *nr = 8; *lanes = 16; *threads = 128; }
  else { *nr = 16; *lanes = 16; *threads = 128; }
}

// Floats of scratch the walk wants per (row, head): three staged rows.
KF_API int kf_delta_rule_row_floats(int d) {
  int nr, lanes, threads;
  delta_shape(d, &nr, &lanes, &threads);
  return 3 * lanes * (nr == 4 ? 4 : nr + 4);
}

// d up to 256 key channels, any dv.  Rows of single-token steps and of prompt portions run the same two kernels.
// prep: T * H * kf_delta_rule_row_floats(d) floats (16-byte aligned); small: T * H * 2 floats.
KF_API int kf_delta_rule(const float* qkv, int ld_qkv, int q0, int k0, int v0, const float* beta, int ld_beta, int beta0,
                         const float* decay, int ld_decay, int decay0, int per_channel, const void* dt_bias, const void* a_log,
                         int w_dtype, float* state, float* out, int ld_out, int H, int KH, int d, int dv, int n_reqs,
                         const int* req_row_start, const int* req_n_rows, const int* req_state_slot, int writes, int T,
                         float* prep, float* small, cudaStream_t stream) {
  if (n_reqs <= 0 || T <= 0) return KF_OK;
  if (d < 1 || d > 256 || dv < 1 || H < 1 || KH < 1 || H % KH) return KF_ERR_SIZE;
  if (!prep || !small || ((uintptr_t)prep & 15)) return KF_ERR_ALIGN;
  KfDeltaArgs p{qkv, ld_qkv, q0, k0, v0, beta, ld_beta, beta0, decay, ld_decay, decay0, per_channel, dt_bias, a_log,
                state, out, ld_out, H, KH, d, dv, n_reqs, req_row_start, req_n_rows, req_state_slot, writes};
  int nr, lanes, threads;
  delta_shape(d, &nr, &lanes, &threads);
  const dim3 pgrid(kf_ceil_div((long)T * H, 4));
  if (w_dtype == KF_F32) kf_launch(delta_prepare_kernel<float>, pgrid, dim3(128), 0, stream, p, prep, small, T, nr, lanes);
  else if (w_dtype == KF_BF16) kf_launch(delta_prepare_kernel<__nv_bfloat16>, pgrid, dim3(128), 0, stream, p, prep, small, T, nr, lanes);
  else return KF_ERR_DTYPE;
  KF_CHECK_LAUNCH();
  const dim3 grid(n_reqs * H, kf_ceil_div(dv, threads / lanes));
  if (d <= 32) kf_launch(delta_rule_kernel<8, 4, 128>, grid, dim3(128), 0, stream, p, (const float*)prep, (const float*)small);
  else if (d <= 64) kf_launch(delta_rule_kernel<8, 8, 128>, grid, dim3(128), 0, stream, p, (const float*)prep, (const float*)small);
  else if (d <= 128) kf_launch(delta_rule_kernel<8, 16, 128>, grid, dim3(128), 0, stream, p, (const float*)prep, (const float*)small);
  else kf_launch(delta_rule_kernel<16, 16, 128>, grid, dim3(128), 0, stream, p, (const float*)prep, (const float*)small);
  KF_CHECK_LAUNCH();
  return KF_OK;
}

// out[t, h*dv + i] = o[t, h*dv + i] / sqrt(mean_i(o[t, h, :]^2) + eps) * w[i] * act(gate[t, gate0 + h*dv + i]),
// act: 0 = silu, 1 = sigmoid.  One warp per (row, head).
template <typename TW, typename TO>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const TW* __restrict__ w, float eps,
                                      const float* __restrict__ gate, int ld_gate, int gate0, int act,
                                      TO* __restrict__ out, int H, int dv, int T, int w_stride, int ldo, int ocol0, float scale) {
  kf_pdl_trigger();
  kf_pdl_wait();
  const int lane = threadIdx.x & 31;
  const long item = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long)T * H) return;
  const int t = (int)(item / H), h = (int)(item - (long)t * H);
  const float* src = o + ((size_t)t * H + h) * dv;
  float ss = 0.f;
  for (int i = lane; i < dv; i += 32) ss = fmaf(src[i], src[i], ss);
  ss = kf_warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)dv + eps);
  const float* g = gate + (size_t)t * ld_gate + gate0 + h * dv;
  for (int i = lane; i < dv; i += 32) {
    const float z = g[i];
    const float s = 1.f / (1.f + expf(-z));
    kf_store(out, (size_t)t * ldo + ocol0 + h * dv + i, src[i] * inv * kf_load(w, h * w_stride + i) * (act == 0 ? z * s : s) * scale);
  }
}

KF_API int kf_head_norm_gate(const float* o, const void* w, int w_dtype, float eps, const float* gate, int ld_gate, int gate0,
                             int act, void* out, int out_dtype, int H, int dv, int T, int w_stride, int ldo, int ocol0, float scale,
                             cudaStream_t stream) {
  if (T <= 0) return KF_OK;
  if (ldo <= 0) ldo = H * dv;                   // rows of `out` hold the heads alone
  if (ocol0 < 0 || ocol0 + H * dv > ldo) return KF_ERR_SIZE;
  const dim3 grid(kf_ceil_div((long)T * H, 4));
#define KF_GO(TW, TO) \
  kf_launch(head_norm_gate_kernel<TW, TO>, grid, dim3(128), 0, stream, o, (const TW*)w, eps, gate, ld_gate, gate0, act, (TO*)out, H, dv, T, w_stride, ldo, ocol0, scale)
  if (w_dtype == KF_F32 && out_dtype == KF_F32) KF_GO(float, float);
  else if (w_dtype == KF_BF16 && out_dtype == KF_BF16) KF_GO(__nv_bfloat16, __nv_bfloat16);
  else if (w_dtype == KF_BF16 && out_dtype == KF_F32) KF_GO(__nv_bfloat16, float);
  else if (w_dtype == KF_F32 && out_dtype == KF_BF16) KF_GO(float, __nv_bfloat16);
  else return KF_ERR_DTYPE;
#undef KF_GO
  KF_CHECK_LAUNCH();
  return KF_OK;
}
