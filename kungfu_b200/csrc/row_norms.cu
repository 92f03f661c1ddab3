// Root-mean-square norms in groups, and the polynomial activation that norms its powers.
//
// A row of H elements is cut into `groups` equal consecutive parts; each part is divided by its own
// sqrt(mean(part^2) + eps) and the whole row is multiplied by a weight vector:
//   group_rmsnorm:      out[r, :] = gnorm(x[row(r), :]) * w
//   add_group_rmsnorm:  x += gnorm(a) * w1 (a may be absent);  x += shift (a vector, may be absent);
//                       optionally out2 = gnorm(x) * w2        (post-norm + residual + a constant row + next pre-norm)
// A block owns one (row, part): both norms of the second kernel cut the row alike, so a part never needs another
// part's values.  A part of up to NPT * blockDim elements stays in registers between its sums and its stores.
//
//   poly_norm:  out = a N(z) + b N(z^2) + c N(z^3) + e,  N(u) = u / sqrt(mean(u^2) + eps) over the row, powers element by
//               element; the four numbers come from a tensor.  One block per row, the three sums in one pass.
// Sums and factors are 32-bit; only the stores round.
#include "common.cuh"

constexpr int GN_NPT = 8;

template <typename TW, typename TO, bool REG>
__global__ void group_rmsnorm_kernel(const float* __restrict__ x, const TW* __restrict__ w, float eps, int part,
                                     TO* __restrict__ out, const int* __restrict__ rows, int H) {
  kf_pdl_trigger();
  kf_pdl_wait();
  __shared__ float red[33];
  const int r = blockIdx.x, c0 = blockIdx.y * part;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * H + c0;
  TO* o = out + (size_t)r * H + c0;
  float v[REG ? GN_NPT : 1];
  float ss = 0.f;
  if (REG) {
#pragma unroll
    for (int k = 0; k < GN_NPT; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      v[k] = i < part ? xr[i] : 0.f;
      ss = fmaf(v[k], v[k], ss);
    }
  } else {
    for (int i = threadIdx.x; i < part; i += blockDim.x) ss = fmaf(xr[i], xr[i], ss);
  }
  ss = kf_block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)part + eps);
  if (REG) {
#pragma unroll
    for (int k = 0; k < GN_NPT; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      if (i < part) kf_store(o, i, v[k] * inv * kf_load(w, c0 + i));
    }
  } else {
    for (int i = threadIdx.x; i < part; i += blockDim.x) kf_store(o, i, xr[i] * inv * kf_load(w, c0 + i));
  }
}

template <typename TW, typename TO, bool REG>
__global__ void add_group_rmsnorm_kernel(const float* __restrict__ a, const TW* __restrict__ w1, float eps1, float* __restrict__ x,
                                         const TW* __restrict__ shift, const TW* __restrict__ w2, float eps2,
                                         TO* __restrict__ out2, int part, int H) {
  kf_pdl_trigger();
  kf_pdl_wait();
  __shared__ float red[33];
  const int r = blockIdx.x, c0 = blockIdx.y * part;
  const float* ar = a ? a + (size_t)r * H + c0 : nullptr;
  float* xr = x + (size_t)r * H + c0;
  float v[REG ? GN_NPT : 1];
  float inv = 0.f;
  if (ar) {
    float ss = 0.f;
    if (REG) {
#pragma unroll
      for (int k = 0; k < GN_NPT; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        v[k] = i < part ? ar[i] : 0.f;
        ss = fmaf(v[k], v[k], ss);
      }
    } else {
      for (int i = threadIdx.x; i < part; i += blockDim.x) ss = fmaf(ar[i], ar[i], ss);
    }
    ss = kf_block_sum(ss, red);
    inv = 1.f / sqrtf(ss / (float)part + eps1);
  }
  float ss2 = 0.f;
  if (REG) {
#pragma unroll
    for (int k = 0; k < GN_NPT; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      if (i < part) {
        float y = xr[i];
        if (ar) y += v[k] * inv * kf_load(w1, c0 + i);
        if (shift) y += kf_load(shift, c0 + i);
        xr[i] = y;
        v[k] = y;
        ss2 = fmaf(y, y, ss2);
      }
    }
  } else {
    for (int i = threadIdx.x; i < part; i += blockDim.x) {
      float y = xr[i];
      if (ar) y += ar[i] * inv * kf_load(w1, c0 + i);
      if (shift) y += kf_load(shift, c0 + i);
      xr[i] = y;
      ss2 = fmaf(y, y, ss2);
    }
  }
  if (out2 == nullptr) return;
  ss2 = kf_block_sum(ss2, red);
  const float inv2 = 1.f / sqrtf(ss2 / (float)part + eps2);
  TO* o = out2 + (size_t)r * H + c0;
  if (REG) {
#pragma unroll
    for (int k = 0; k < GN_NPT; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      if (i < part) kf_store(o, i, v[k] * inv2 * kf_load(w2, c0 + i));
    }
  } else {
    for (int i = threadIdx.x; i < part; i += blockDim.x) kf_store(o, i, xr[i] * inv2 * kf_load(w2, c0 + i));   // own writes
  }
}

static inline int gn_threads(int part) {
  int t = (part + GN_NPT - 1) / GN_NPT;
  t = (t + 31) / 32 * 32;
  return t < 32 ? 32 : (t > 512 ? 512 : t);
}

KF_API int kf_group_rmsnorm(const float* x, const void* w, int w_dtype, float eps, int groups, void* out, int out_dtype,
                            const int* rows, int n, int H, cudaStream_t stream) {
  if (n <= 0) return KF_OK;
  if (groups < 1 || H % groups) return KF_ERR_SIZE;
  const int part = H / groups, threads = gn_threads(part);
  const bool reg = part <= GN_NPT * threads;
#define KF_GO(TW, TO)                                                                                                     \
  do {                                                                                                                    \
    if (reg) kf_launch(group_rmsnorm_kernel<TW, TO, true>, dim3(n, groups), dim3(threads), 0, stream, x, (const TW*)w, eps, part, (TO*)out, rows, H); \
    else kf_launch(group_rmsnorm_kernel<TW, TO, false>, dim3(n, groups), dim3(threads), 0, stream, x, (const TW*)w, eps, part, (TO*)out, rows, H);    \
  } while (0)
  if (w_dtype == KF_F32 && out_dtype == KF_F32) KF_GO(float, float);
  else if (w_dtype == KF_BF16 && out_dtype == KF_BF16) KF_GO(__nv_bfloat16, __nv_bfloat16);
  else if (w_dtype == KF_BF16 && out_dtype == KF_F32) KF_GO(__nv_bfloat16, float);
  else if (w_dtype == KF_F32 && out_dtype == KF_BF16) KF_GO(float, __nv_bfloat16);
  else return KF_ERR_DTYPE;
#undef KF_GO
  KF_CHECK_LAUNCH();
  return KF_OK;
}

// a, shift, w2/out2 may each be null; w1, shift and w2 share one element type.
KF_API int kf_add_group_rmsnorm(const float* a, const void* w1, int w_dtype, float eps1, float* x, const void* shift,
                                const void* w2, float eps2, void* out2, int out_dtype, int groups, int T, int H,
                                cudaStream_t stream) {
  if (T <= 0) return KF_OK;
  if (groups < 1 || H % groups || (a && !w1) || (out2 && !w2)) return KF_ERR_SIZE;
  const int part = H / groups, threads = gn_threads(part);
  const bool reg = part <= GN_NPT * threads;
#define KF_GO(TW, TO)                                                                                                     \
  do {                                                                                                                    \
    if (reg) kf_launch(add_group_rmsnorm_kernel<TW, TO, true>, dim3(T, groups), dim3(threads), 0, stream, a, (const TW*)w1, eps1, x, \
                       (const TW*)shift, (const TW*)w2, eps2, (TO*)out2, part, H);                                        \
    else kf_launch(add_group_rmsnorm_kernel<TW, TO, false>, dim3(T, groups), dim3(threads), 0, stream, a, (const TW*)w1, eps1, x,    \
                   (const TW*)shift, (const TW*)w2, eps2, (TO*)out2, part, H);                                            \
  } while (0)
  if (w_dtype == KF_F32 && out_dtype == KF_F32) KF_GO(float, float);
  else if (w_dtype == KF_BF16 && out_dtype == KF_BF16) KF_GO(__nv_bfloat16, __nv_bfloat16);
  else if (w_dtype == KF_BF16 && out_dtype == KF_F32) KF_GO(__nv_bfloat16, float);
  else if (w_dtype == KF_F32 && out_dtype == KF_BF16) KF_GO(float, __nv_bfloat16);
  else return KF_ERR_DTYPE;
#undef KF_GO
  KF_CHECK_LAUNCH();
  return KF_OK;
}

// Three sums of a block at once; every thread gets them.  `red` holds 3 * 33 floats.
__device__ __forceinline__ void kf_block_sum3(float& a, float& b, float& c, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  a = kf_warp_sum(a); b = kf_warp_sum(b); c = kf_warp_sum(c);
  if (lane == 0) { red[warp] = a; red[33 + warp] = b; red[66 + warp] = c; }
  __syncthreads();
  if (warp == 0) {
    float ta = lane < nwarp ? red[lane] : 0.f, tb = lane < nwarp ? red[33 + lane] : 0.f, tc = lane < nwarp ? red[66 + lane] : 0.f;
    ta = kf_warp_sum(ta); tb = kf_warp_sum(tb); tc = kf_warp_sum(tc);
    if (lane == 0) { red[32] = ta; red[65] = tb; red[98] = tc; }
  }
  __syncthreads();
  a = red[32]; b = red[65]; c = red[98];
}

constexpr int PN_NPT = 8;

template <typename TW, typename TO, bool REG>
__global__ void poly_norm_kernel(const float* __restrict__ z, const TW* __restrict__ coef, float eps, TO* __restrict__ out, int I) {
  kf_pdl_trigger();
  const float ca = kf_load(coef, 0), cb = kf_load(coef, 1), cc = kf_load(coef, 2), ce = kf_load(coef, 3);
  kf_pdl_wait();
  __shared__ float red[99];
  const float* zr = z + (size_t)blockIdx.x * I;
  TO* o = out + (size_t)blockIdx.x * I;
  float v[REG ? PN_NPT : 1];
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  if (REG) {
#pragma unroll
    for (int k = 0; k < PN_NPT; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      v[k] = i < I ? zr[i] : 0.f;
      const float q = v[k] * v[k];
      s2 += q; s4 = fmaf(q, q, s4); s6 = fmaf(q * q, q, s6);
    }
  } else {
    for (int i = threadIdx.x; i < I; i += blockDim.x) {
      const float q = zr[i] * zr[i];
      s2 += q; s4 = fmaf(q, q, s4); s6 = fmaf(q * q, q, s6);
    }
  }
  kf_block_sum3(s2, s4, s6, red);
  const float n = (float)I;
  const float i1 = ca / sqrtf(s2 / n + eps), i2 = cb / sqrtf(s4 / n + eps), i3 = cc / sqrtf(s6 / n + eps);
  if (REG) {
#pragma unroll
    for (int k = 0; k < PN_NPT; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      const float u = v[k];
      if (i < I) kf_store(o, i, fmaf(u * u * u, i3, fmaf(u * u, i2, fmaf(u, i1, ce))));
    }
  } else {
    for (int i = threadIdx.x; i < I; i += blockDim.x) {
      const float u = zr[i];
      kf_store(o, i, fmaf(u * u * u, i3, fmaf(u * u, i2, fmaf(u, i1, ce))));
    }
  }
}

KF_API int kf_poly_norm(const float* z, const void* coef, int w_dtype, float eps, void* out, int out_dtype, int T, int I,
                        cudaStream_t stream) {
  if (T <= 0) return KF_OK;
  if (I < 1) return KF_ERR_SIZE;
  int threads = ((I + PN_NPT - 1) / PN_NPT + 31) / 32 * 32;
  threads = threads < 64 ? 64 : (threads > 1024 ? 1024 : threads);
  const bool reg = I <= PN_NPT * threads;
#define KF_GO(TW, TO)                                                                                                   \
  do {                                                                                                                  \
    if (reg) kf_launch(poly_norm_kernel<TW, TO, true>, dim3(T), dim3(threads), 0, stream, z, (const TW*)coef, eps, (TO*)out, I); \
    else kf_launch(poly_norm_kernel<TW, TO, false>, dim3(T), dim3(threads), 0, stream, z, (const TW*)coef, eps, (TO*)out, I);    \
  } while (0)
  if (w_dtype == KF_F32 && out_dtype == KF_F32) KF_GO(float, float);
  else if (w_dtype == KF_BF16 && out_dtype == KF_BF16) KF_GO(__nv_bfloat16, __nv_bfloat16);
  else if (w_dtype == KF_BF16 && out_dtype == KF_F32) KF_GO(__nv_bfloat16, float);
  else if (w_dtype == KF_F32 && out_dtype == KF_BF16) KF_GO(float, __nv_bfloat16);
  else return KF_ERR_DTYPE;
#undef KF_GO
  KF_CHECK_LAUNCH();
  return KF_OK;
}
