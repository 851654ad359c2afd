// Training-side kernels for sm_100a (all HBM-bound, single pass, 16-byte accesses):
//
//   logprob_entropy_fwd / _bwd : per-token log-probability of a target and (optionally) the
//       entropy straight from a chunk of fp32 logits, and the matching gradient written as
//       bf16 dlogits. Together with the chunked lm_head GEMM this replaces the reference's
//       log_softmax over [B,T,V] (rollouts/training/losses.py:98-124, 171-175, 216-226).
//   rmsnorm_bwd                : dx and per-CTA partial dw of RMSNorm.
//   rope_fwd / rope_bwd        : rotate_half RoPE on [T,H,D] (backward = rotation by -angle).
//   adamw                      : fp32 master weights + moments, bf16 or fp32 grads, optional
//                                clip coefficient read from device memory, bf16 param write-back.
//   sumsq_partial              : per-CTA partial sums of squares for the global grad norm
//                                (replaces one .norm().item() per parameter,
//                                rollouts/training/backends/fsdp.py:398-419).
#include "common.cuh"

namespace rb {

constexpr int ROW_THREADS = 512;

struct Lse { float m, s; };
__device__ __forceinline__ Lse lse_merge(Lse a, Lse b) {
  const float m = fmaxf(a.m, b.m);
  if (m == -INFINITY) return {m, 0.f};
  return {m, a.s * __expf(a.m - m) + b.s * __expf(b.m - m)};
}
__device__ __forceinline__ Lse block_lse(Lse v) {
  __shared__ float sm_m[ROW_THREADS / 32], sm_s[ROW_THREADS / 32];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Lse other = {__shfl_xor_sync(0xffffffffu, v.m, o), __shfl_xor_sync(0xffffffffu, v.s, o)};
    v = lse_merge(v, other);
  }
  if (lane == 0) { sm_m[wid] = v.m; sm_s[wid] = v.s; }
  __syncthreads();
  Lse r = {lane < ROW_THREADS / 32 ? sm_m[lane] : -INFINITY, lane < ROW_THREADS / 32 ? sm_s[lane] : 0.f};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Lse other = {__shfl_xor_sync(0xffffffffu, r.m, o), __shfl_xor_sync(0xffffffffu, r.s, o)};
    r = lse_merge(r, other);
  }
  __syncthreads();
  return r;
}
__device__ __forceinline__ float block_sum(float v) {
  __shared__ float sm[ROW_THREADS / 32];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  v = warp_sum(v);
  if (lane == 0) sm[wid] = v;
  __syncthreads();
  float r = lane < (blockDim.x >> 5) ? sm[lane] : 0.f;
  r = warp_sum(r);
  __syncthreads();
  return r;
}

// One CTA per row. entropy may be null. Targets < 0 (ignored positions) give logprob 0.
__global__ void __launch_bounds__(ROW_THREADS)
logprob_entropy_fwd_kernel(const float* __restrict__ logits, long long ld, int V, const int* __restrict__ targets,
                           float* __restrict__ logprob, float* __restrict__ lse_out, float* __restrict__ entropy) {
  const long long row = blockIdx.x;
  const float* x = logits + row * ld;
  Lse v = {-INFINITY, 0.f};
  for (int i = threadIdx.x; i < V; i += ROW_THREADS) v = lse_merge(v, {x[i], 1.f});
  v = block_lse(v);
  const float lse = v.m + __logf(v.s);
  float ent = 0.f;
  if (entropy != nullptr) {
    float acc = 0.f;
    for (int i = threadIdx.x; i < V; i += ROW_THREADS) {
      const float lp = x[i] - lse;
      acc -= __expf(lp) * lp;
    }
    ent = block_sum(acc);
  }
  if (threadIdx.x == 0) {
    const int t = targets[row];
    logprob[row] = (t >= 0 && t < V) ? x[t] - lse : 0.f;
    lse_out[row] = lse;
    if (entropy != nullptr) entropy[row] = ent;
  }
}

// dlogits[j] = g_lp * (1[j == t] - p_j) - g_ent * p_j * (log p_j + H)
__global__ void __launch_bounds__(ROW_THREADS)
logprob_entropy_bwd_kernel(const float* __restrict__ logits, long long ld, int V, const int* __restrict__ targets,
                           const float* __restrict__ lse, const float* __restrict__ entropy,
                           const float* __restrict__ g_logprob, const float* __restrict__ g_entropy,
                           __nv_bfloat16* __restrict__ dlogits, long long ldd) {
  const long long row = blockIdx.x;
  const float* x = logits + row * ld;
  __nv_bfloat16* d = dlogits + row * ldd;
  const int t = targets[row];
  const float glp = (t >= 0 && t < V) ? g_logprob[row] : 0.f;
  const float gent = g_entropy != nullptr ? g_entropy[row] : 0.f;
  const float H = entropy != nullptr ? entropy[row] : 0.f;
  const float l = lse[row];
  for (int i = threadIdx.x * 2; i < V; i += ROW_THREADS * 2) {
    float o[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int c = i + j;
      if (c < V) {
        const float lp = x[c] - l;
        const float p = __expf(lp);
        o[j] = glp * ((c == t ? 1.f : 0.f) - p) - gent * p * (lp + H);
      } else {
        o[j] = 0.f;
      }
    }
    if (i + 1 < V && ((ldd & 1) == 0)) {
      *reinterpret_cast<uint32_t*>(d + i) = pack_bf16x2(o[0], o[1]);
    } else {
      d[i] = __float2bfloat16_rn(o[0]);
      if (i + 1 < V) d[i + 1] = __float2bfloat16_rn(o[1]);
    }
  }
}

// ------------------------------------------------------------------------------------------
// RMSNorm backward. y = w * xhat, xhat = x * rstd.  dx = rstd * (g - xhat * mean(g * xhat)),
// g = dy * w. dw partials: one row of [gridDim.x, d] fp32 per CTA (summed by the caller).
// ------------------------------------------------------------------------------------------
__global__ void rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                   const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dx,
                                   float* __restrict__ dw_partial, long long rows, int d, float eps) {
  extern __shared__ float dw_acc[];  // [d]
  for (int i = threadIdx.x; i < d; i += blockDim.x) dw_acc[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (long long row = (long long)blockIdx.x * nw + wid; row < rows; row += (long long)gridDim.x * nw) {
    const __nv_bfloat16* xr = x + row * d;
    const __nv_bfloat16* gr = dy + row * d;
    float ss = 0.f, dot = 0.f;
    for (int i = lane; i < d; i += 32) {
      const float xv = __bfloat162float(xr[i]);
      ss += xv * xv;
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)d + eps);
    for (int i = lane; i < d; i += 32) {
      const float xh = __bfloat162float(xr[i]) * rstd;
      const float g = __bfloat162float(gr[i]) * __bfloat162float(w[i]);
      dot += g * xh;
    }
    dot = warp_sum(dot) / (float)d;
    for (int i = lane; i < d; i += 32) {
      const float xh = __bfloat162float(xr[i]) * rstd;
      const float dyv = __bfloat162float(gr[i]);
      const float g = dyv * __bfloat162float(w[i]);
      dx[row * d + i] = __float2bfloat16_rn(rstd * (g - xh * dot));
      atomicAdd(&dw_acc[i], dyv * xh);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < d; i += blockDim.x) dw_partial[(long long)blockIdx.x * d + i] = dw_acc[i];
}

// Same result for d <= 1024, d % 8 == 0 (wider rows would spill): one warp per row, the row of x and dy read once with 16-byte loads and
// kept in registers (VPL vectors of 8 values per lane), the weight-gradient contribution of all rows a warp
// handles accumulated in registers and merged into shared memory once at the end.
template <int VPL>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_vec_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                       const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dx,
                       float* __restrict__ dw_partial, long long rows, int d, float eps) {
  extern __shared__ float dw_acc[];  // [d]
  for (int i = threadIdx.x; i < d; i += blockDim.x) dw_acc[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int nvec = d >> 3;
  float wv[VPL][8], dwv[VPL][8];
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const int v = lane + 32 * j;
    uint4 q = make_uint4(0, 0, 0, 0);
    if (v < nvec) q = *reinterpret_cast<const uint4*>(w + v * 8);
    const uint32_t qi[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = unpack_bf16x2(qi[e]);
      wv[j][2 * e] = f.x; wv[j][2 * e + 1] = f.y;
      dwv[j][2 * e] = 0.f; dwv[j][2 * e + 1] = 0.f;
    }
  }
  for (long long row = (long long)blockIdx.x * nw + wid; row < rows; row += (long long)gridDim.x * nw) {
    float xs[VPL][8], gs[VPL][8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int v = lane + 32 * j;
      uint4 a = make_uint4(0, 0, 0, 0), b = make_uint4(0, 0, 0, 0);
      if (v < nvec) {
        a = *reinterpret_cast<const uint4*>(x + row * d + v * 8);
        b = *reinterpret_cast<const uint4*>(dy + row * d + v * 8);
      }
      const uint32_t ai[4] = {a.x, a.y, a.z, a.w}, bi[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 fa = unpack_bf16x2(ai[e]), fb = unpack_bf16x2(bi[e]);
        xs[j][2 * e] = fa.x; xs[j][2 * e + 1] = fa.y;
        gs[j][2 * e] = fb.x; gs[j][2 * e + 1] = fb.y;
        ss = fmaf(fa.x, fa.x, ss); ss = fmaf(fa.y, fa.y, ss);
      }
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)d + eps);
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j)
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        xs[j][e] *= rstd;                                   // xhat
        dot = fmaf(gs[j][e] * wv[j][e], xs[j][e], dot);
      }
    dot = warp_sum(dot) / (float)d;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int v = lane + 32 * j;
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float g0 = gs[j][2 * e] * wv[j][2 * e], g1 = gs[j][2 * e + 1] * wv[j][2 * e + 1];
        o[e] = pack_bf16x2(rstd * (g0 - xs[j][2 * e] * dot), rstd * (g1 - xs[j][2 * e + 1] * dot));
        dwv[j][2 * e] = fmaf(gs[j][2 * e], xs[j][2 * e], dwv[j][2 * e]);
        dwv[j][2 * e + 1] = fmaf(gs[j][2 * e + 1], xs[j][2 * e + 1], dwv[j][2 * e + 1]);
      }
      if (v < nvec) *reinterpret_cast<uint4*>(dx + row * d + v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const int v = lane + 32 * j;
    if (v < nvec)
#pragma unroll
      for (int e = 0; e < 8; ++e) atomicAdd(&dw_acc[v * 8 + e], dwv[j][e]);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < d; i += blockDim.x) dw_partial[(long long)blockIdx.x * d + i] = dw_acc[i];
}

// Wide rows (1024 < d <= 8192, d % 8 == 0): one CTA of 256 threads per row at a time. Thread t owns the 16-byte
// vectors t, t + 256, ... of every row it sees, so x and dy are read once into registers, the two row sums
// (sum x^2 and sum dy*w*x) share one block reduction, and the weight-gradient contribution of all rows of the CTA
// accumulates in registers (the columns of a thread never change): no shared-memory atomics.
template <int VPT>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_wide_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                        const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dx,
                        float* __restrict__ dw_partial, long long rows, int d, float eps) {
  __shared__ float red[2][8];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int nvec = d >> 3;
  float wv[VPT][8], dwv[VPT][8];
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int v = threadIdx.x + 256 * j;
    uint4 q = make_uint4(0, 0, 0, 0);
    if (v < nvec) q = *reinterpret_cast<const uint4*>(w + v * 8);
    const uint32_t qi[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = unpack_bf16x2(qi[e]);
      wv[j][2 * e] = f.x; wv[j][2 * e + 1] = f.y;
      dwv[j][2 * e] = 0.f; dwv[j][2 * e + 1] = 0.f;
    }
  }
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    float xs[VPT][8], gs[VPT][8];
    float ss = 0.f, gwx = 0.f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int v = threadIdx.x + 256 * j;
      uint4 a = make_uint4(0, 0, 0, 0), b = make_uint4(0, 0, 0, 0);
      if (v < nvec) {
        a = *reinterpret_cast<const uint4*>(x + row * d + v * 8);
        b = *reinterpret_cast<const uint4*>(dy + row * d + v * 8);
      }
      const uint32_t ai[4] = {a.x, a.y, a.z, a.w}, bi[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 fa = unpack_bf16x2(ai[e]), fb = unpack_bf16x2(bi[e]);
        xs[j][2 * e] = fa.x; xs[j][2 * e + 1] = fa.y;
        gs[j][2 * e] = fb.x; gs[j][2 * e + 1] = fb.y;
        ss = fmaf(fa.x, fa.x, ss); ss = fmaf(fa.y, fa.y, ss);
        gwx = fmaf(fb.x * wv[j][2 * e], fa.x, gwx); gwx = fmaf(fb.y * wv[j][2 * e + 1], fa.y, gwx);
      }
    }
    ss = warp_sum(ss);
    gwx = warp_sum(gwx);
    __syncthreads();   // the previous row's sums have been read by every warp
    if (lane == 0) { red[0][wid] = ss; red[1][wid] = gwx; }
    __syncthreads();
    float tss = 0.f, tg = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) { tss += red[0][k]; tg += red[1][k]; }
    const float rstd = rsqrtf(tss / (float)d + eps);
    const float dot = tg * rstd / (float)d;     // mean over the row of (dy * w) * xhat
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int v = threadIdx.x + 256 * j;
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float xh0 = xs[j][2 * e] * rstd, xh1 = xs[j][2 * e + 1] * rstd;
        const float g0 = gs[j][2 * e] * wv[j][2 * e], g1 = gs[j][2 * e + 1] * wv[j][2 * e + 1];
        o[e] = pack_bf16x2(rstd * (g0 - xh0 * dot), rstd * (g1 - xh1 * dot));
        dwv[j][2 * e] = fmaf(gs[j][2 * e], xh0, dwv[j][2 * e]);
        dwv[j][2 * e + 1] = fmaf(gs[j][2 * e + 1], xh1, dwv[j][2 * e + 1]);
      }
      if (v < nvec) *reinterpret_cast<uint4*>(dx + row * d + v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int v = threadIdx.x + 256 * j;
    if (v < nvec) {
      float* dst = dw_partial + (long long)blockIdx.x * d + v * 8;
      *reinterpret_cast<float4*>(dst) = make_float4(dwv[j][0], dwv[j][1], dwv[j][2], dwv[j][3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(dwv[j][4], dwv[j][5], dwv[j][6], dwv[j][7]);
    }
  }
}

// ------------------------------------------------------------------------------------------
// RoPE on [T, H, D] (training: no cache). sign = +1 forward, -1 backward (inverse rotation).
// fp32 math, one rounding at the end.
// ------------------------------------------------------------------------------------------
__global__ void rope_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                            const int* __restrict__ positions, const float2* __restrict__ cos_sin, long long T, int H,
                            int D, long long ldx, long long ldy, int max_pos, float sign) {
  const int half = D >> 1;
  const long long n = T * H * half;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int j = (int)(i % half);
    const long long th = i / half;
    const int h = (int)(th % H);
    const long long t = th / H;
    int pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
    const float2 cs = cos_sin[(long long)pos * half + j];
    const float s = cs.y * sign;
    const __nv_bfloat16* xr = x + t * ldx + (long long)h * D;
    __nv_bfloat16* yr = y + t * ldy + (long long)h * D;
    const float lo = __bfloat162float(xr[j]), hi = __bfloat162float(xr[j + half]);
    yr[j] = __float2bfloat16_rn(lo * cs.x - hi * s);
    yr[j + half] = __float2bfloat16_rn(hi * cs.x + lo * s);
  }
}

// Same rotation with 16-byte accesses: one thread rotates eight (lo, hi) pairs of one head. Needs D / 2 to be a
// multiple of 8 and 16-byte aligned rows (x, y, row strides, the table).
__global__ void rope_vec8_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                 const int* __restrict__ positions, const float2* __restrict__ cos_sin, long long T, int H,
                                 int D, long long ldx, long long ldy, int max_pos, float sign) {
  const int half = D >> 1, groups = half >> 3;
  const long long n = T * H * groups;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int j = (int)(i % groups) * 8;
    const long long th = i / groups;
    const int h = (int)(th % H);
    const long long t = th / H;
    int pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
    const float4* cs4 = reinterpret_cast<const float4*>(cos_sin + (long long)pos * half + j);
    const __nv_bfloat16* xr = x + t * ldx + (long long)h * D + j;
    __nv_bfloat16* yr = y + t * ldy + (long long)h * D + j;
    const uint4 lo4 = *reinterpret_cast<const uint4*>(xr), hi4 = *reinterpret_cast<const uint4*>(xr + half);
    const uint32_t lo_w[4] = {lo4.x, lo4.y, lo4.z, lo4.w}, hi_w[4] = {hi4.x, hi4.y, hi4.z, hi4.w};
    uint32_t olo[4], ohi[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float4 cs = cs4[e];   // (cos, sin) of two consecutive rotation pairs
      const float2 lo = unpack_bf16x2(lo_w[e]), hi = unpack_bf16x2(hi_w[e]);
      const float s0 = cs.y * sign, s1 = cs.w * sign;
      olo[e] = pack_bf16x2(lo.x * cs.x - hi.x * s0, lo.y * cs.z - hi.y * s1);
      ohi[e] = pack_bf16x2(hi.x * cs.x + lo.x * s0, hi.y * cs.z + lo.y * s1);
    }
    *reinterpret_cast<uint4*>(yr) = make_uint4(olo[0], olo[1], olo[2], olo[3]);
    *reinterpret_cast<uint4*>(yr + half) = make_uint4(ohi[0], ohi[1], ohi[2], ohi[3]);
  }
}

// ------------------------------------------------------------------------------------------
// Sum of squares partials and AdamW
// ------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename G>
__global__ void sumsq_partial_kernel(const G* __restrict__ g, long long n, float scale, float* __restrict__ partial) {
  float acc = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = to_f<G>(g[i]) * scale;
    acc += v * v;
  }
  acc = block_sum(acc);
  if (threadIdx.x == 0) partial[blockIdx.x] = acc;
}

// clip_coef: device pointer to min(1, max_norm / (norm + 1e-6)) or null.
template <typename G>
__global__ void adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                             const G* __restrict__ grad, __nv_bfloat16* __restrict__ param_bf16, long long n, float lr,
                             float beta1, float beta2, float eps, float weight_decay, float bc1, float bc2,
                             float grad_scale, const float* __restrict__ clip_coef) {
  const float clip = clip_coef != nullptr ? *clip_coef : 1.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float g = to_f<G>(grad[i]) * grad_scale * clip;
    float p = master[i];
    const float mi = beta1 * m[i] + (1.f - beta1) * g;
    const float vi = beta2 * v[i] + (1.f - beta2) * g * g;
    m[i] = mi;
    v[i] = vi;
    p = p * (1.f - lr * weight_decay) - lr * (mi / bc1) / (sqrtf(vi / bc2) + eps);
    master[i] = p;
    if (param_bf16 != nullptr) param_bf16[i] = __float2bfloat16_rn(p);
  }
}

// out (bf16 or fp32) += in (bf16), used for gradient accumulation buffers.
__global__ void accumulate_kernel(float* __restrict__ acc, const __nv_bfloat16* __restrict__ in, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    acc[i] += __bfloat162float(in[i]);
}

}  // namespace rb

using namespace rb;
#define RB_OK() (cudaGetLastError() == cudaSuccess ? 0 : -11)
static inline unsigned grid_for(long long n, int threads, int cap = 148 * 16) {
  long long g = (n + threads - 1) / threads;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (unsigned)g;
}

extern "C" int rb_logprob_entropy_fwd(const float* logits, long long ld, int rows, int V, const int* targets,
                                      float* logprob, float* lse, float* entropy, cudaStream_t s) {
  if (rows <= 0) return 0;
  logprob_entropy_fwd_kernel<<<rows, ROW_THREADS, 0, s>>>(logits, ld, V, targets, logprob, lse, entropy);
  return RB_OK();
}
extern "C" int rb_logprob_entropy_bwd(const float* logits, long long ld, int rows, int V, const int* targets,
                                      const float* lse, const float* entropy, const float* g_logprob,
                                      const float* g_entropy, void* dlogits, long long ldd, cudaStream_t s) {
  if (rows <= 0) return 0;
  logprob_entropy_bwd_kernel<<<rows, ROW_THREADS, 0, s>>>(logits, ld, V, targets, lse, entropy, g_logprob, g_entropy,
                                                         (__nv_bfloat16*)dlogits, ldd);
  return RB_OK();
}
extern "C" int rb_rmsnorm_bwd_num_partials() { return 148 * 2; }
extern "C" int rb_rmsnorm_bwd(const void* x, const void* w, const void* dy, void* dx, float* dw_partial,
                              long long rows, int d, float eps, cudaStream_t s) {
  if (rows <= 0) return 0;
  const int grid = rb_rmsnorm_bwd_num_partials();
  const __nv_bfloat16 *xb = (const __nv_bfloat16*)x, *wb = (const __nv_bfloat16*)w, *gb = (const __nv_bfloat16*)dy;
  const bool vec = d % 8 == 0 && d <= 1024 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) |
                                                reinterpret_cast<uintptr_t>(dx) | reinterpret_cast<uintptr_t>(w)) & 15) == 0;
  const size_t sm = d * sizeof(float);
  const bool wide = d % 8 == 0 && d > 1024 && d <= 8192 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) |
                    reinterpret_cast<uintptr_t>(dx) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(dw_partial)) & 15) == 0;
  if (wide) {
    if (d <= 2048) rmsnorm_bwd_wide_kernel<1><<<grid, 256, 0, s>>>(xb, wb, gb, (__nv_bfloat16*)dx, dw_partial, rows, d, eps);
    else if (d <= 4096) rmsnorm_bwd_wide_kernel<2><<<grid, 256, 0, s>>>(xb, wb, gb, (__nv_bfloat16*)dx, dw_partial, rows, d, eps);
    else rmsnorm_bwd_wide_kernel<4><<<grid, 256, 0, s>>>(xb, wb, gb, (__nv_bfloat16*)dx, dw_partial, rows, d, eps);
    return RB_OK();
  }
  if (!vec) rmsnorm_bwd_kernel<<<grid, 256, sm, s>>>(xb, wb, gb, (__nv_bfloat16*)dx, dw_partial, rows, d, eps);
  else if (d <= 256) rmsnorm_bwd_vec_kernel<1><<<grid, 256, sm, s>>>(xb, wb, gb, (__nv_bfloat16*)dx, dw_partial, rows, d, eps);
  else if (d <= 512) rmsnorm_bwd_vec_kernel<2><<<grid, 256, sm, s>>>(xb, wb, gb, (__nv_bfloat16*)dx, dw_partial, rows, d, eps);
  else rmsnorm_bwd_vec_kernel<4><<<grid, 256, sm, s>>>(xb, wb, gb, (__nv_bfloat16*)dx, dw_partial, rows, d, eps);
  return RB_OK();
}
extern "C" int rb_rope(const void* x, void* y, const int* positions, const void* cos_sin, long long T, int H, int D,
                       long long ldx, long long ldy, int max_pos, int backward, cudaStream_t s) {
  if (T <= 0) return 0;
  const long long n = T * H * (D / 2);
  const bool vec = (D % 16 == 0) && ldx % 8 == 0 && ldy % 8 == 0 &&
                   ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(cos_sin)) & 15) == 0;
  if (vec)
    rope_vec8_kernel<<<grid_for(n / 8, 256), 256, 0, s>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, positions,
                                                          (const float2*)cos_sin, T, H, D, ldx, ldy, max_pos,
                                                          backward ? -1.f : 1.f);
  else
    rope_kernel<<<grid_for(n, 256), 256, 0, s>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, positions,
                                                 (const float2*)cos_sin, T, H, D, ldx, ldy, max_pos,
                                                 backward ? -1.f : 1.f);
  return RB_OK();
}
extern "C" int rb_sumsq_num_partials() { return 148 * 4; }
extern "C" int rb_sumsq_partial(const void* g, long long n, int grad_is_f32, float scale, float* partial,
                                cudaStream_t s) {
  const int grid = rb_sumsq_num_partials();
  if (grad_is_f32) sumsq_partial_kernel<float><<<grid, ROW_THREADS, 0, s>>>((const float*)g, n, scale, partial);
  else sumsq_partial_kernel<__nv_bfloat16><<<grid, ROW_THREADS, 0, s>>>((const __nv_bfloat16*)g, n, scale, partial);
  return RB_OK();
}
extern "C" int rb_adamw(float* master, float* m, float* v, const void* grad, int grad_is_f32, void* param_bf16,
                        long long n, float lr, float beta1, float beta2, float eps, float weight_decay, int step,
                        float grad_scale, const float* clip_coef, cudaStream_t s) {
  if (n <= 0) return 0;
  const float bc1 = 1.f - powf(beta1, (float)step), bc2 = 1.f - powf(beta2, (float)step);
  const unsigned grid = grid_for(n, 256, 148 * 8);
  if (grad_is_f32)
    adamw_kernel<float><<<grid, 256, 0, s>>>(master, m, v, (const float*)grad, (__nv_bfloat16*)param_bf16, n, lr, beta1,
                                             beta2, eps, weight_decay, bc1, bc2, grad_scale, clip_coef);
  else
    adamw_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(master, m, v, (const __nv_bfloat16*)grad,
                                                     (__nv_bfloat16*)param_bf16, n, lr, beta1, beta2, eps, weight_decay,
                                                     bc1, bc2, grad_scale, clip_coef);
  return RB_OK();
}
extern "C" int rb_accumulate_f32_bf16(float* acc, const void* in, long long n, cudaStream_t s) {
  if (n <= 0) return 0;
  accumulate_kernel<<<grid_for(n, 256), 256, 0, s>>>(acc, (const __nv_bfloat16*)in, n);
  return RB_OK();
}

// ------------------------------------------------------------------------------------------
// Small activation / normalisation kernels of the dev experiments (dev/speedrun/single-file.py:786-787,
// 973-975, 1140: relu^2 MLP, logit soft-capping; dev/integration-evaluation: row log-softmax forward and
// backward). Elementwise ones stream bf16 with 16-byte accesses; log-softmax keeps one row per warp.
// ------------------------------------------------------------------------------------------
namespace rb {

// mode 0: y = relu(x)^2          backward: dx = 2 relu(x) dy
// mode 1: y = cap * tanh(x/cap)  backward: dx = (1 - tanh(x/cap)^2) dy
template <bool BWD>
__global__ void unary_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                             __nv_bfloat16* __restrict__ out, long long n, int mode, float cap) {
  const long long nvec = n >> 3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const uint4 xv = reinterpret_cast<const uint4*>(x)[i];
    uint4 gv = make_uint4(0, 0, 0, 0);
    if (BWD) gv = reinterpret_cast<const uint4*>(dy)[i];
    const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w}, gs[4] = {gv.x, gv.y, gv.z, gv.w};
    uint32_t os[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = unpack_bf16x2(xs[j]), g = unpack_bf16x2(gs[j]);
      float r[2];
      const float in[2] = {a.x, a.y}, gg[2] = {g.x, g.y};
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (mode == 0) {
          const float p = fmaxf(in[t], 0.f);
          r[t] = BWD ? 2.f * p * gg[t] : p * p;
        } else {
          const float th = tanhf(in[t] / cap);
          r[t] = BWD ? (1.f - th * th) * gg[t] : cap * th;
        }
      }
      os[j] = pack_bf16x2(r[0], r[1]);
    }
    reinterpret_cast<uint4*>(out)[i] = make_uint4(os[0], os[1], os[2], os[3]);
  }
}

// y[r, :] = x[r, :] - logsumexp(x[r, :])   (fp32 in / out), one warp per row
__global__ void log_softmax_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, int rows, int cols) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  const float* xr = x + (long long)row * cols;
  float m = -INFINITY, s = 0.f;
  for (int c = lane; c < cols; c += 32) {
    const float v = xr[c];
    if (v > m) { s *= __expf(m - v); m = v; }
    s += __expf(v - m);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    const float mn = fmaxf(m, m2);
    s = (mn == -INFINITY) ? 0.f : s * __expf(m - mn) + s2 * __expf(m2 - mn);
    m = mn;
  }
  const float lse = m + __logf(s);
  for (int c = lane; c < cols; c += 32) y[(long long)row * cols + c] = xr[c] - lse;
}

// dx = dy - exp(y) * sum(dy)
__global__ void log_softmax_bwd_kernel(const float* __restrict__ y, const float* __restrict__ dy, float* __restrict__ dx,
                                       int rows, int cols) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  const long long base = (long long)row * cols;
  float s = 0.f;
  for (int c = lane; c < cols; c += 32) s += dy[base + c];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  for (int c = lane; c < cols; c += 32) dx[base + c] = dy[base + c] - __expf(y[base + c]) * s;
}

}  // namespace rb

extern "C" int rb_unary(const void* x, const void* dy, void* out, long long n, int mode, float cap, cudaStream_t s) {
  if (n <= 0) return 0;
  if (n % 8 != 0 || mode < 0 || mode > 1 || (mode == 1 && cap <= 0.f)) return -1;
  long long grid = ((n >> 3) + 255) / 256;
  if (grid > 148 * 16) grid = 148 * 16;
  if (dy == nullptr)
    rb::unary_kernel<false><<<(unsigned)grid, 256, 0, s>>>((const __nv_bfloat16*)x, nullptr, (__nv_bfloat16*)out, n, mode, cap);
  else
    rb::unary_kernel<true><<<(unsigned)grid, 256, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, (__nv_bfloat16*)out, n, mode, cap);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int rb_log_softmax(const float* x, const float* dy, float* out, int rows, int cols, cudaStream_t s) {
  if (rows <= 0 || cols <= 0) return 0;
  const unsigned grid = (rows + 7) / 8;
  if (dy == nullptr) rb::log_softmax_fwd_kernel<<<grid, 256, 0, s>>>(x, out, rows, cols);
  else rb::log_softmax_bwd_kernel<<<grid, 256, 0, s>>>(x, dy, out, rows, cols);     // x is y (the forward output) here
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// ------------------------------------------------------------------------------------------
// Adaptive average pooling over [N, C, H, W] fp32 (dev/integration-evaluation/_adaptive_avg_pool2d*.py) and a
// 16-byte vector add (dev/kernel-learning/leetgpu/vector-addition). Pooling window of output o along an axis of
// length L pooled to O cells: [floor(o L / O), ceil((o + 1) L / O)). The backward gathers: every input element
// sums dy / window size over the output cells whose window contains it, so no atomics are needed.
// ------------------------------------------------------------------------------------------
namespace rb {
__device__ __forceinline__ int pool_lo(int o, int L, int O) { return (int)(((long long)o * L) / O); }
__device__ __forceinline__ int pool_hi(int o, int L, int O) { return (int)((((long long)(o + 1)) * L + O - 1) / O); }

__global__ void adaptive_avg_pool2d_kernel(const float* __restrict__ x, float* __restrict__ y, long long planes, int H, int W,
                                           int OH, int OW) {
  const long long n = planes * OH * OW;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int ow = (int)(i % OW), oh = (int)((i / OW) % OH);
    const long long pl = i / ((long long)OW * OH);
    const int h0 = pool_lo(oh, H, OH), h1 = pool_hi(oh, H, OH), w0 = pool_lo(ow, W, OW), w1 = pool_hi(ow, W, OW);
    float acc = 0.f;
    for (int h = h0; h < h1; ++h)
      for (int w = w0; w < w1; ++w) acc += x[(pl * H + h) * W + w];
    y[i] = acc / (float)((h1 - h0) * (w1 - w0));
  }
}
__global__ void adaptive_avg_pool2d_bwd_kernel(const float* __restrict__ dy, float* __restrict__ dx, long long planes, int H,
                                               int W, int OH, int OW) {
  const long long n = planes * H * W;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int w = (int)(i % W), h = (int)((i / W) % H);
    const long long pl = i / ((long long)W * H);
    // output cells whose window can contain h lie in (h OH / H - 1, (h + 1) OH / H); one spare cell on each side,
    // the containment test below decides
    const int oh_a = max((int)(((long long)h * OH) / H) - 1, 0), oh_b = min((int)((((long long)h + 1) * OH + H - 1) / H) + 1, OH);
    const int ow_a = max((int)(((long long)w * OW) / W) - 1, 0), ow_b = min((int)((((long long)w + 1) * OW + W - 1) / W) + 1, OW);
    float acc = 0.f;
    for (int oh = oh_a; oh < oh_b; ++oh) {
      const int h0 = pool_lo(oh, H, OH), h1 = pool_hi(oh, H, OH);
      if (h < h0 || h >= h1) continue;
      for (int ow = ow_a; ow < ow_b; ++ow) {
        const int w0 = pool_lo(ow, W, OW), w1 = pool_hi(ow, W, OW);
        if (w < w0 || w >= w1) continue;
        acc += dy[(pl * OH + oh) * OW + ow] / (float)((h1 - h0) * (w1 - w0));
      }
    }
    dx[i] = acc;
  }
}
__global__ void vec_add_bf16_kernel(const uint4* __restrict__ a, const uint4* __restrict__ b, uint4* __restrict__ c, long long nvec) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const uint4 x = a[i], y = b[i];
    const uint32_t xi[4] = {x.x, x.y, x.z, x.w}, yi[4] = {y.x, y.y, y.z, y.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(xi[j]), g = unpack_bf16x2(yi[j]);
      o[j] = pack_bf16x2(f.x + g.x, f.y + g.y);
    }
    c[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}
}  // namespace rb

extern "C" int rb_adaptive_avg_pool2d(const float* x, const float* dy, float* out, long long planes, int H, int W, int OH, int OW,
                                      cudaStream_t s) {
  if (planes <= 0 || H <= 0 || W <= 0 || OH <= 0 || OW <= 0) return -1;
  if (dy == nullptr) {
    rb::adaptive_avg_pool2d_kernel<<<grid_for(planes * OH * OW, 256), 256, 0, s>>>(x, out, planes, H, W, OH, OW);
  } else {
    rb::adaptive_avg_pool2d_bwd_kernel<<<grid_for(planes * H * W, 256), 256, 0, s>>>(dy, out, planes, H, W, OH, OW);
  }
  return RB_OK();
}
extern "C" int rb_vec_add_bf16(const void* a, const void* b, void* c, long long n, cudaStream_t s) {
  if (n <= 0 || n % 8 != 0) return -1;
  rb::vec_add_bf16_kernel<<<grid_for(n / 8, 256), 256, 0, s>>>((const uint4*)a, (const uint4*)b, (uint4*)c, n / 8);
  return RB_OK();
}
