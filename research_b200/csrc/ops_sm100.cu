// Memory-bound transformer ops for sm_100a: RMSNorm (row and per-head), RoPE fused with the
// paged KV-cache append, SwiGLU, embedding gather, seeded sampling with log-probabilities.
// All kernels are single-pass over HBM with 16-byte accesses; rounding points follow the
// bf16 Hugging Face modules (see the functional oracles in research_b200/models/functional.py)
// so that greedy decoding matches the fp32/bf16 reference token for token.
#include "common.cuh"

namespace rb {

// ------------------------------------------------------------------------------------------
// RMSNorm: y = bf16( bf16(x * rsqrt(mean(x^2)+eps)) * w ). One warp per row.
// Reference math: rollouts/tools/functional_extractor/qwen_functional.py:46-65.
// ------------------------------------------------------------------------------------------
// The row is read from global memory once: up to 8 vectors of 8 bf16 per lane stay in
// registers (d <= 2048); longer rows fall back to a second read that hits L1/L2.
__global__ void rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                               __nv_bfloat16* __restrict__ y, long long rows, int d, long long ldx,
                               long long ldy, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int MAXV = 8;
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const __nv_bfloat16* xr = x + row * ldx;
  __nv_bfloat16* yr = y + row * ldy;
  const int nvec = d >> 3;
  const bool in_regs = nvec <= MAXV * 32;
  uint4 keep[MAXV];
  float ss = 0.f;
  if (in_regs) {
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = lane + 32 * i;
      keep[i] = v < nvec ? *reinterpret_cast<const uint4*>(xr + v * 8) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      float2 f;
      f = unpack_bf16x2(keep[i].x); ss += f.x * f.x + f.y * f.y;
      f = unpack_bf16x2(keep[i].y); ss += f.x * f.x + f.y * f.y;
      f = unpack_bf16x2(keep[i].z); ss += f.x * f.x + f.y * f.y;
      f = unpack_bf16x2(keep[i].w); ss += f.x * f.x + f.y * f.y;
    }
  } else {
    for (int v = lane; v < nvec; v += 32) {
      uint4 u = *reinterpret_cast<const uint4*>(xr + v * 8);
      float2 f;
      f = unpack_bf16x2(u.x); ss += f.x * f.x + f.y * f.y;
      f = unpack_bf16x2(u.y); ss += f.x * f.x + f.y * f.y;
      f = unpack_bf16x2(u.z); ss += f.x * f.x + f.y * f.y;
      f = unpack_bf16x2(u.w); ss += f.x * f.x + f.y * f.y;
    }
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / (float)d + eps);
  auto emit = [&](int v, uint4 u) {
    uint4 ww = *reinterpret_cast<const uint4*>(w + v * 8);
    uint32_t xi[4] = {u.x, u.y, u.z, u.w};
    uint32_t wi[4] = {ww.x, ww.y, ww.z, ww.w};
    uint32_t oi[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = unpack_bf16x2(xi[j]);
      float2 g = unpack_bf16x2(wi[j]);
      // round the normalised value to bf16 before the weight multiply, like the HF module
      float a = __bfloat162float(__float2bfloat16_rn(f.x * rstd));
      float b = __bfloat162float(__float2bfloat16_rn(f.y * rstd));
      oi[j] = pack_bf16x2(a * g.x, b * g.y);
    }
    *reinterpret_cast<uint4*>(yr + v * 8) = make_uint4(oi[0], oi[1], oi[2], oi[3]);
  };
  if (in_regs) {
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) emit(v, keep[i]);
    }
  } else {
    for (int v = lane; v < nvec; v += 32) emit(v, *reinterpret_cast<const uint4*>(xr + v * 8));
  }
}

// ------------------------------------------------------------------------------------------
// RoPE (rotate_half convention) + optional per-head QK RMSNorm + paged KV append.
//   qkv   : [T, (Hq + 2*Hkv) * D] bf16  (q heads, then k heads, then v heads)
//   q_out : [T, Hq * D] bf16 (rotated)
//   k_cache / v_cache : [num_blocks, Hkv, block_size, D] bf16, slot = block*block_size + off
//   cos_sin : [max_pos, D/2] float2
// One warp per (token, head). Slots < 0 are skipped (padding rows of a captured graph).
// Reference math: qwen_functional.py:68-150; cache store: inference/attention/flex_backend.py:116-142.
// ------------------------------------------------------------------------------------------
template <int D>
__global__ void rope_kv_append_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out,
                                      __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                      const int* __restrict__ positions, const int* __restrict__ slots,
                                      const float2* __restrict__ cos_sin, const __nv_bfloat16* __restrict__ q_norm_w,
                                      const __nv_bfloat16* __restrict__ k_norm_w, float norm_eps, int T, int Hq,
                                      int Hkv, int block_size, long long num_slots, int max_pos, int* status) {
  constexpr int HALF = D / 2;
  constexpr int PER_LANE = HALF / 32;  // pairs handled per lane: D=64 -> 1, D=128 -> 2
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long gw = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int heads = Hq + 2 * Hkv;
  if (gw >= (long long)T * heads) return;
  const int t = (int)(gw / heads);
  const int h = (int)(gw % heads);
  const __nv_bfloat16* src = qkv + (long long)t * heads * D + (long long)h * D;
  int pos = positions[t];
  const int slot = slots[t];
  if (pos < 0) pos = 0;
  if (pos >= max_pos) { set_status(status, ST_BAD_INDEX); pos = max_pos - 1; }

  float lo[PER_LANE], hi[PER_LANE];
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    lo[j] = __bfloat162float(src[lane + 32 * j]);
    hi[j] = __bfloat162float(src[lane + 32 * j + HALF]);
  }
  __nv_bfloat16* dst;
  bool is_v = h >= Hq + Hkv;
  if (h < Hq) {
    dst = q_out + (long long)t * Hq * D + (long long)h * D;
  } else {
    if (slot < 0) return;
    if (slot >= num_slots) { set_status(status, ST_BAD_INDEX); return; }
    const int kvh = is_v ? h - Hq - Hkv : h - Hq;
    const long long blk = slot / block_size, off = slot % block_size;
    __nv_bfloat16* cache = is_v ? v_cache : k_cache;
    dst = cache + ((blk * Hkv + kvh) * block_size + off) * D;
  }
  if (is_v) {
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) {
      dst[lane + 32 * j] = __float2bfloat16_rn(lo[j]);
      dst[lane + 32 * j + HALF] = __float2bfloat16_rn(hi[j]);
    }
    return;
  }
  const __nv_bfloat16* nw = (h < Hq) ? q_norm_w : k_norm_w;
  if (nw != nullptr) {
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) ss += lo[j] * lo[j] + hi[j] * hi[j];
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)D + norm_eps);
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) {
      float a = __bfloat162float(__float2bfloat16_rn(lo[j] * rstd));
      float b = __bfloat162float(__float2bfloat16_rn(hi[j] * rstd));
      lo[j] = __bfloat162float(__float2bfloat16_rn(a * __bfloat162float(nw[lane + 32 * j])));
      hi[j] = __bfloat162float(__float2bfloat16_rn(b * __bfloat162float(nw[lane + 32 * j + HALF])));
    }
  }
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    const float2 cs = cos_sin[(long long)pos * HALF + lane + 32 * j];
    // bf16 rounding of cos/sin and of each product mirrors q*cos + rotate_half(q)*sin in bf16
    const float c = __bfloat162float(__float2bfloat16_rn(cs.x));
    const float s = __bfloat162float(__float2bfloat16_rn(cs.y));
    const float a = __bfloat162float(__float2bfloat16_rn(lo[j] * c));
    const float b = __bfloat162float(__float2bfloat16_rn(-hi[j] * s));
    const float e = __bfloat162float(__float2bfloat16_rn(hi[j] * c));
    const float f = __bfloat162float(__float2bfloat16_rn(lo[j] * s));
    dst[lane + 32 * j] = __float2bfloat16_rn(a + b);
    dst[lane + 32 * j + HALF] = __float2bfloat16_rn(e + f);
  }
}

// ------------------------------------------------------------------------------------------
// SwiGLU: out = bf16( bf16(silu(gate)) * up ), gate|up packed as [T, 2F].
// Reference math: qwen_functional.py:251-274.
// ------------------------------------------------------------------------------------------
// `rows_dev` (optional) bounds the row count from device memory: the expert-parallel MoE layer only knows on the
// device how many routed rows it received.
__global__ void swiglu_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                              long long T, int F, const int* __restrict__ rows_dev) {
  pdl_launch_dependents();
  pdl_wait();
  if (rows_dev != nullptr) {
    const long long r = *rows_dev;
    T = r < T ? (r < 0 ? 0 : r) : T;
  }
  const long long nvec = T * (F >> 3);
  const int fv = F >> 3;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / fv;
    const int c = (int)(i % fv) * 8;
    uint4 g = *reinterpret_cast<const uint4*>(gu + t * 2 * F + c);
    uint4 u = *reinterpret_cast<const uint4*>(gu + t * 2 * F + F + c);
    uint32_t gi[4] = {g.x, g.y, g.z, g.w}, ui[4] = {u.x, u.y, u.z, u.w}, oi[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 a = unpack_bf16x2(gi[j]);
      float2 b = unpack_bf16x2(ui[j]);
      float s0 = __bfloat162float(__float2bfloat16_rn(a.x / (1.f + __expf(-a.x))));
      float s1 = __bfloat162float(__float2bfloat16_rn(a.y / (1.f + __expf(-a.y))));
      oi[j] = pack_bf16x2(s0 * b.x, s1 * b.y);
    }
    *reinterpret_cast<uint4*>(out + t * F + c) = make_uint4(oi[0], oi[1], oi[2], oi[3]);
  }
}

// SwiGLU backward: given gate|up [T,2F] and dout [T,F] writes dgate|dup [T,2F].
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dout,
                                  __nv_bfloat16* __restrict__ dgu, long long T, int F) {
  // 8 columns (16 bytes) per thread and step; F % 8 == 0 is checked by the launcher
  const int fv = F >> 3;
  const long long nvec = T * fv;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / fv;
    const int c = (int)(i % fv) * 8;
    const uint4 g4 = *reinterpret_cast<const uint4*>(gu + t * 2 * F + c);
    const uint4 u4 = *reinterpret_cast<const uint4*>(gu + t * 2 * F + F + c);
    const uint4 d4 = *reinterpret_cast<const uint4*>(dout + t * F + c);
    const uint32_t gi[4] = {g4.x, g4.y, g4.z, g4.w}, ui[4] = {u4.x, u4.y, u4.z, u4.w}, di[4] = {d4.x, d4.y, d4.z, d4.w};
    uint32_t og[4], ou[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 g = unpack_bf16x2(gi[j]), u = unpack_bf16x2(ui[j]), dy = unpack_bf16x2(di[j]);
      const float s0 = 1.f / (1.f + __expf(-g.x)), s1 = 1.f / (1.f + __expf(-g.y));
      const float l0 = g.x * s0, l1 = g.y * s1;
      og[j] = pack_bf16x2(dy.x * u.x * (s0 + l0 * (1.f - s0)), dy.y * u.y * (s1 + l1 * (1.f - s1)));
      ou[j] = pack_bf16x2(dy.x * l0, dy.y * l1);
    }
    *reinterpret_cast<uint4*>(dgu + t * 2 * F + c) = make_uint4(og[0], og[1], og[2], og[3]);
    *reinterpret_cast<uint4*>(dgu + t * 2 * F + F + c) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
  }
}

// ------------------------------------------------------------------------------------------
// Embedding gather: out[t, :] = table[ids[t], :]
// ------------------------------------------------------------------------------------------
__global__ void embedding_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                 __nv_bfloat16* __restrict__ out, int T, int d, int vocab, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  if (t >= T) return;
  int id = ids[t];
  if (id < 0 || id >= vocab) { if (threadIdx.x == 0) set_status(status, ST_BAD_INDEX); id = 0; }
  const uint4* src = reinterpret_cast<const uint4*>(table + (long long)id * d);
  uint4* dst = reinterpret_cast<uint4*>(out + (long long)t * d);
  for (int v = threadIdx.x; v < (d >> 3); v += blockDim.x) dst[v] = src[v];
}

// ------------------------------------------------------------------------------------------
// Sampling with log-probabilities, one CTA per row of fp32 logits [B, V].
//   token  ~ softmax(logits / T)   via the Gumbel-max trick with a counter-based RNG
//            (temperature == 0 -> argmax)
//   logprob = log_softmax(logits)[token]  from the UNSCALED logits (true policy probability)
// Reference behaviour: rollouts/inference/sampling.py:10-58.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
  // splitmix64 finaliser: turns (seed, step) into the per-row key once per CTA
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
__device__ __forceinline__ uint32_t hash32(uint32_t idx, uint32_t k0, uint32_t k1) {
  // counter-based 32-bit mixer (murmur3 finaliser) - every (row key, column) has its own draw
  uint32_t h = (idx * 0x9E3779B1u) ^ k0;
  h ^= h >> 16; h *= 0x85EBCA6Bu;
  h ^= h >> 13; h *= 0xC2B2AE35u;
  h ^= h >> 16;
  return h + k1;
}

constexpr int SAMPLE_THREADS = 512;

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_logprob_kernel(const float* __restrict__ logits, long long ld, int V,
                      const float* __restrict__ temperature, const unsigned long long* __restrict__ seeds,
                      const unsigned long long* __restrict__ step_ptr, unsigned long long step_add,
                      int* __restrict__ out_tokens, float* __restrict__ out_logprobs,
                      float4* __restrict__ partials /*[rows][splits], splits > 1 only*/, int* __restrict__ tickets /*[rows]*/) {
  pdl_launch_dependents();
  pdl_wait();
  // grid (splits, rows): with few rows the vocabulary of a row is cut into `splits` contiguous chunks so that all
  // SMs share the transcendental work (three per element); the last CTA of a row merges the chunk records in
  // chunk order
  const int splits = gridDim.x;
  const int chunk = (((V + splits - 1) / splits) + 3) & ~3;
  const int v_lo = blockIdx.x * chunk;
  const int v_hi = min(V, v_lo + chunk);
  // The step counter lives in device memory so a captured CUDA graph draws fresh noise on
  // every replay (the host bumps the counter between replays).
  const unsigned long long step = step_add + (step_ptr != nullptr ? *step_ptr : 0ull);
  const int row = blockIdx.y;
  const float* lr = logits + (long long)row * ld;
  const float temp = temperature[row];
  const bool greedy = temp <= 0.f;
  const float inv_t = greedy ? 1.f : 1.f / temp;
  const uint64_t key = mix64(mix64(seeds[row]) ^ (step * 0x9E3779B97F4A7C15ull));
  const uint32_t k0 = (uint32_t)key, k1 = (uint32_t)(key >> 32);

  float m = -INFINITY, ssum = 0.f;     // online log-sum-exp of the unscaled logits
  float best = -INFINITY;              // best perturbed score
  int best_i = 0x7fffffff;
  const bool vec_ok = ((ld & 3) == 0) && ((reinterpret_cast<uintptr_t>(lr) & 15) == 0);
  for (int i = v_lo + threadIdx.x * 4; i < v_hi; i += SAMPLE_THREADS * 4) {
    float v[4];
    if (i + 3 < v_hi && vec_ok) {
      float4 f = __ldcs(reinterpret_cast<const float4*>(lr + i));
      v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = (i + j < v_hi) ? lr[i + j] : -INFINITY;
    }
    // one rescale of the running sum per 4 elements instead of a branch per element
    const float m4 = fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3]));
    if (m4 > m) { ssum *= __expf(m - m4); m = m4; }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float x = v[j];          // -inf past the end: contributes exp(-inf) = 0
      ssum += __expf(x - m);
      float score = x * inv_t;
      if (!greedy) {
        const uint32_t r = hash32((uint32_t)(i + j), k0, k1);
        const float u = ((float)(r >> 8) + 0.5f) * (1.0f / 16777216.0f);  // (0,1)
        // Gumbel noise -ln(-ln u) with two fast log2 (ln x = log2 x * ln 2)
        score -= 0.6931471805599453f * __log2f(-0.6931471805599453f * __log2f(u));
      }
      if (score > best) { best = score; best_i = i + j; }
    }
  }
  // block reduction
  __shared__ float sm_m[SAMPLE_THREADS / 32], sm_s[SAMPLE_THREADS / 32], sm_b[SAMPLE_THREADS / 32];
  __shared__ int sm_i[SAMPLE_THREADS / 32];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    const float s2 = __shfl_xor_sync(0xffffffffu, ssum, o);
    const float b2 = __shfl_xor_sync(0xffffffffu, best, o);
    const int i2 = __shfl_xor_sync(0xffffffffu, best_i, o);
    const float mn = fmaxf(m, m2);
    ssum = (mn == -INFINITY) ? 0.f : ssum * __expf(m - mn) + s2 * __expf(m2 - mn);
    m = mn;
    if (b2 > best || (b2 == best && i2 < best_i)) { best = b2; best_i = i2; }
  }
  if (lane == 0) { sm_m[wid] = m; sm_s[wid] = ssum; sm_b[wid] = best; sm_i[wid] = best_i; }
  __syncthreads();
  if (wid == 0) {
    constexpr int NW = SAMPLE_THREADS / 32;
    m = lane < NW ? sm_m[lane] : -INFINITY;
    ssum = lane < NW ? sm_s[lane] : 0.f;
    best = lane < NW ? sm_b[lane] : -INFINITY;
    best_i = lane < NW ? sm_i[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
      const float s2 = __shfl_xor_sync(0xffffffffu, ssum, o);
      const float b2 = __shfl_xor_sync(0xffffffffu, best, o);
      const int i2 = __shfl_xor_sync(0xffffffffu, best_i, o);
      const float mn = fmaxf(m, m2);
      ssum = (mn == -INFINITY) ? 0.f : ssum * __expf(m - mn) + s2 * __expf(m2 - mn);
      m = mn;
      if (b2 > best || (b2 == best && i2 < best_i)) { best = b2; best_i = i2; }
    }
    if (lane == 0) {
      if (splits > 1) {
        partials[(long long)row * splits + blockIdx.x] = make_float4(m, ssum, best, __int_as_float(best_i));
        __threadfence();
        const int tk = atomicAdd(&tickets[row], 1);
        if (tk != splits - 1) return;
        tickets[row] = 0;           // ready for the next launch
        __threadfence();
        m = -INFINITY; ssum = 0.f; best = -INFINITY; best_i = 0x7fffffff;
        for (int c = 0; c < splits; ++c) {   // chunk order: the sums do not depend on which CTA finished last
          const float4 r = __ldcg(&partials[(long long)row * splits + c]);
          const int i2 = __float_as_int(r.w);
          const float mn = fmaxf(m, r.x);
          ssum = (mn == -INFINITY) ? 0.f : ssum * __expf(m - mn) + r.y * __expf(r.x - mn);
          m = mn;
          if (r.z > best || (r.z == best && i2 < best_i)) { best = r.z; best_i = i2; }
        }
      }
      if (best_i >= V) best_i = 0;
      out_tokens[row] = best_i;
      out_logprobs[row] = lr[best_i] - (m + __logf(ssum));
    }
  }
}

// Per-token log-probability of given tokens from fp32 logits (teacher forcing / verification).
__global__ void __launch_bounds__(SAMPLE_THREADS)
token_logprob_kernel(const float* __restrict__ logits, long long ld, int V, const int* __restrict__ tokens,
                     float* __restrict__ out_logprobs) {
  const int row = blockIdx.x;
  const float* lr = logits + (long long)row * ld;
  float m = -INFINITY, ssum = 0.f;
  for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) {
    const float x = lr[i];
    if (x > m) { ssum = ssum * __expf(m - x) + 1.f; m = x; } else { ssum += __expf(x - m); }
  }
  __shared__ float sm_m[SAMPLE_THREADS / 32], sm_s[SAMPLE_THREADS / 32];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    const float s2 = __shfl_xor_sync(0xffffffffu, ssum, o);
    const float mn = fmaxf(m, m2);
    ssum = (mn == -INFINITY) ? 0.f : ssum * __expf(m - mn) + s2 * __expf(m2 - mn);
    m = mn;
  }
  if (lane == 0) { sm_m[wid] = m; sm_s[wid] = ssum; }
  __syncthreads();
  if (wid == 0) {
    constexpr int NW = SAMPLE_THREADS / 32;
    m = lane < NW ? sm_m[lane] : -INFINITY;
    ssum = lane < NW ? sm_s[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
      const float s2 = __shfl_xor_sync(0xffffffffu, ssum, o);
      const float mn = fmaxf(m, m2);
      ssum = (mn == -INFINITY) ? 0.f : ssum * __expf(m - mn) + s2 * __expf(m2 - mn);
      m = mn;
    }
    if (lane == 0) {
      int tok = tokens[row];
      if (tok < 0 || tok >= V) tok = 0;
      out_logprobs[row] = lr[tok] - (m + __logf(ssum));
    }
  }
}

// bf16 2-D transpose (used by the training path when an operand must change majorness).
__global__ void transpose_bf16_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                      int rows, int cols) {
  __shared__ __nv_bfloat16 tile[32][33];
  int x = blockIdx.x * 32 + threadIdx.x;
  int y0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int y = y0 + j;
    if (x < cols && y < rows) tile[j][threadIdx.x] = in[(long long)y * cols + x];
  }
  __syncthreads();
  int ox = blockIdx.y * 32 + threadIdx.x;
  int oy0 = blockIdx.x * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int oy = oy0 + j;
    if (ox < rows && oy < cols) out[(long long)oy * rows + ox] = tile[threadIdx.x][j];
  }
}

}  // namespace rb

using namespace rb;

#define RB_CHECK_LAUNCH() (cudaGetLastError() == cudaSuccess ? 0 : -11)

extern "C" void rb_ops_set_pdl(int on) { rb::pdl_enabled() = on != 0; }

extern "C" int rb_rmsnorm(const void* x, const void* w, void* y, long long rows, int d, long long ldx,
                          long long ldy, float eps, cudaStream_t stream) {
  if (d % 8 != 0 || rows <= 0) return -1;
  const int warps = rows >= 148 * 8 * 4 ? 8 : 2;   // few rows: spread them over more SMs
  const long long grid = (rows + warps - 1) / warps;
  return launch_kernel(rmsnorm_kernel, dim3((unsigned)grid), dim3(warps * 32), 0, stream, (const __nv_bfloat16*)x,
                       (const __nv_bfloat16*)w, (__nv_bfloat16*)y, rows, d, ldx, ldy, eps) == cudaSuccess ? 0 : -11;
}

extern "C" int rb_rope_kv_append(const void* qkv, void* q_out, void* k_cache, void* v_cache,
                                 const int* positions, const int* slots, const void* cos_sin,
                                 const void* q_norm_w, const void* k_norm_w, float norm_eps, int T, int Hq,
                                 int Hkv, int D, int block_size, long long num_slots, int max_pos,
                                 int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  const long long warps_total = (long long)T * (Hq + 2 * Hkv);
  const int warps = 8;
  const unsigned grid = (unsigned)((warps_total + warps - 1) / warps);
#define LAUNCH_ROPE(DD)                                                                              \
  launch_kernel(rope_kv_append_kernel<DD>, dim3(grid), dim3(warps * 32), 0, stream,                   \
      (const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, \
      positions, slots, (const float2*)cos_sin, (const __nv_bfloat16*)q_norm_w,                       \
      (const __nv_bfloat16*)k_norm_w, norm_eps, T, Hq, Hkv, block_size, num_slots, max_pos, status)
  cudaError_t e;
  if (D == 64) { e = LAUNCH_ROPE(64); }
  else if (D == 128) { e = LAUNCH_ROPE(128); }
  else return -1;
#undef LAUNCH_ROPE
  return e == cudaSuccess ? 0 : -11;
}

static int swiglu_launch(const void* gu, void* out, long long T, int F, const int* rows_dev, cudaStream_t stream) {
  if (F % 8 != 0 || T <= 0) return -1;
  const long long nvec = T * (F / 8);
  long long grid = (nvec + 255) / 256;
  if (grid > 148 * 16) grid = 148 * 16;
  return launch_kernel(swiglu_kernel, dim3((unsigned)grid), dim3(256), 0, stream, (const __nv_bfloat16*)gu,
                       (__nv_bfloat16*)out, T, F, rows_dev) == cudaSuccess ? 0 : -11;
}
extern "C" int rb_swiglu(const void* gu, void* out, long long T, int F, cudaStream_t stream) {
  return swiglu_launch(gu, out, T, F, nullptr, stream);
}
// At most T rows, and no more than *rows_dev (read on the device when the kernel runs).
extern "C" int rb_swiglu_bounded(const void* gu, void* out, long long T, int F, const int* rows_dev, cudaStream_t stream) {
  return swiglu_launch(gu, out, T, F, rows_dev, stream);
}

extern "C" int rb_swiglu_bwd(const void* gu, const void* dout, void* dgu, long long T, int F,
                             cudaStream_t stream) {
  if (F % 8 != 0 || T <= 0) return -1;
  const long long n = T * (F / 8);
  long long grid = (n + 255) / 256;
  if (grid > 148 * 32) grid = 148 * 32;
  swiglu_bwd_kernel<<<(unsigned)grid, 256, 0, stream>>>((const __nv_bfloat16*)gu, (const __nv_bfloat16*)dout,
                                                       (__nv_bfloat16*)dgu, T, F);
  return RB_CHECK_LAUNCH();
}

extern "C" int rb_embedding(const int* ids, const void* table, void* out, int T, int d, int vocab,
                            int* status, cudaStream_t stream) {
  if (d % 8 != 0 || T <= 0) return -1;
  return launch_kernel(embedding_kernel, dim3(T), dim3(128), 0, stream, ids, (const __nv_bfloat16*)table,
                       (__nv_bfloat16*)out, T, d, vocab, status) == cudaSuccess ? 0 : -11;
}

extern "C" int rb_sample_logprob(const float* logits, long long ld, int B, int V, const float* temperature,
                                 const unsigned long long* seeds, const unsigned long long* step_ptr,
                                 unsigned long long step_add, int* out_tokens, float* out_logprobs,
                                 cudaStream_t stream) {
  if (B <= 0) return 0;
  return launch_kernel(sample_logprob_kernel, dim3(1, B), dim3(SAMPLE_THREADS), 0, stream, logits, ld, V, temperature,
                       seeds, step_ptr, step_add, out_tokens, out_logprobs, (float4*)nullptr, (int*)nullptr) == cudaSuccess ? 0 : -11;
}
// Same with every row's vocabulary cut into `splits` chunks (grid splits x B). `partials` holds B * splits float4
// records, `tickets` B zero-initialised counters (they reset themselves). splits <= 0 picks about four CTAs per SM.
extern "C" int rb_sample_logprob_split(const float* logits, long long ld, int B, int V, const float* temperature,
                                       const unsigned long long* seeds, const unsigned long long* step_ptr,
                                       unsigned long long step_add, int* out_tokens, float* out_logprobs, void* partials,
                                       int* tickets, int splits, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (splits <= 0) splits = (4 * 148 + B - 1) / B;
  if (splits > 8) splits = 8;
  while (splits > 1 && V / splits < 4096) --splits;
  if (splits > 1 && (partials == nullptr || tickets == nullptr)) return -1;
  return launch_kernel(sample_logprob_kernel, dim3(splits, B), dim3(SAMPLE_THREADS), 0, stream, logits, ld, V, temperature,
                       seeds, step_ptr, step_add, out_tokens, out_logprobs, (float4*)partials, tickets) == cudaSuccess ? 0 : -11;
}

extern "C" int rb_token_logprob(const float* logits, long long ld, int B, int V, const int* tokens,
                                float* out_logprobs, cudaStream_t stream) {
  if (B <= 0) return 0;
  token_logprob_kernel<<<B, SAMPLE_THREADS, 0, stream>>>(logits, ld, V, tokens, out_logprobs);
  return RB_CHECK_LAUNCH();
}

extern "C" int rb_transpose_bf16(const void* in, void* out, int rows, int cols, cudaStream_t stream) {
  dim3 grid((cols + 31) / 32, (rows + 31) / 32);
  dim3 block(32, 8);
  transpose_bf16_kernel<<<grid, block, 0, stream>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, rows, cols);
  return RB_CHECK_LAUNCH();
}
