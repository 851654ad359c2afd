// Paged-KV attention for sm_100a.
//
// KV cache layout (per layer): [num_blocks, Hkv, 16, D] bf16, so the 16 tokens of one block
// of one KV head are one contiguous 2 KB (D=64) / 4 KB (D=128) run: a block is the unit the
// kernels stream with 16-byte asynchronous copies. Sequences that share a prefix through the
// radix tree simply list the same physical block ids in their block tables.
//
//   decode  : one CTA per (sequence, KV head, split). All G = Hq/Hkv query heads of the group
//             are rows of one MMA tile, so K/V are read from HBM once per group (no
//             materialised GQA repeat). Each warp streams its own blocks through a 4-stage
//             cp.async ring, keeps an online-softmax state, and the warps (and splits) are
//             merged at the end. The op is HBM-bound: what matters is bytes in flight.
//   prefill : varlen causal attention of new tokens against cached prefix + themselves; one
//             CTA per (sequence, query head, 64-query tile), K/V tiles double-buffered.
//
// Behaviour replaced: rollouts/inference/attention/flex_backend.py:144-279 (SDPA prefill and
// the host-loop gather decode). Numerics oracle: qwen_functional.py:173-248.
#include "common.cuh"
#include "tma_host.h"

#include <stdlib.h>

namespace rb {

constexpr int KV_BLOCK = 16;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Byte offset of 16-byte chunk `c` of row `r` in a tile whose rows hold D bf16, with the low
// three chunk bits XOR-swizzled by the row so ldmatrix reads are bank-conflict free.
template <int D>
__device__ __forceinline__ uint32_t swz(int r, int c) {
  return (uint32_t)(r * (D * 2) + ((c ^ (r & 7)) << 4));
}

// S(16 x 16 keys) += Q(16 x D) K^T for keys [key0, key0+16) of a swizzled K tile.
template <int D>
__device__ __forceinline__ void qk_16x16(float (&s0)[4], float (&s1)[4], const uint32_t (&qf)[D / 16][4],
                                         uint32_t k_smem, int key0, int lane) {
  const int mat = lane >> 3, r = lane & 7;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    uint32_t b0, b1, b2, b3;
    ldsm_x4(k_smem + swz<D>(key0 + (mat >> 1) * 8 + r, 2 * ks + (mat & 1)), b0, b1, b2, b3);
    mma_16816(s0, qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
    mma_16816(s1, qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b2, b3);
  }
}

// O(16 x D) += P(16 x 16 keys) V for keys [key0, key0+16) of a swizzled V tile.
template <int D>
__device__ __forceinline__ void pv_16x16(float (&o)[D / 8][4], uint32_t p0, uint32_t p1, uint32_t p2, uint32_t p3,
                                         uint32_t v_smem, int key0, int lane) {
  const int mat = lane >> 3, r = lane & 7;
#pragma unroll
  for (int dp = 0; dp < D / 16; ++dp) {
    uint32_t b0, b1, b2, b3;
    ldsm_x4_t(v_smem + swz<D>(key0 + (mat & 1) * 8 + r, 2 * dp + (mat >> 1)), b0, b1, b2, b3);
    mma_16816(o[2 * dp], p0, p1, p2, p3, b0, b1);
    mma_16816(o[2 * dp + 1], p0, p1, p2, p3, b2, b3);
  }
}

// Online-softmax update of one 16x16 score tile held as two C fragments. Rows g (c0,c1) and
// g+8 (c2,c3). `valid0/valid1` give, per fragment, which of this thread's two columns are
// inside the sequence / causal range.
struct RowState { float m0, m1, l0, l1; };

template <int D>
__device__ __forceinline__ void softmax_update(float (&s0)[4], float (&s1)[4], RowState& st, float (&o)[D / 8][4],
                                               float scale_log2, uint32_t& p0, uint32_t& p1, uint32_t& p2,
                                               uint32_t& p3) {
  // scores are already masked with -inf where invalid; work in base-2
#pragma unroll
  for (int j = 0; j < 4; ++j) { s0[j] *= scale_log2; s1[j] *= scale_log2; }
  float mx0 = fmaxf(fmaxf(s0[0], s0[1]), fmaxf(s1[0], s1[1]));
  float mx1 = fmaxf(fmaxf(s0[2], s0[3]), fmaxf(s1[2], s1[3]));
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
  const float mn0 = fmaxf(st.m0, mx0), mn1 = fmaxf(st.m1, mx1);
  // a row with nothing valid so far keeps m = -inf; use 0 as the subtraction base then
  const float base0 = (mn0 == -INFINITY) ? 0.f : mn0;
  const float base1 = (mn1 == -INFINITY) ? 0.f : mn1;
  const float corr0 = exp2f(st.m0 - base0), corr1 = exp2f(st.m1 - base1);
  float e00 = exp2f(s0[0] - base0), e01 = exp2f(s0[1] - base0), e10 = exp2f(s1[0] - base0), e11 = exp2f(s1[1] - base0);
  float f00 = exp2f(s0[2] - base1), f01 = exp2f(s0[3] - base1), f10 = exp2f(s1[2] - base1), f11 = exp2f(s1[3] - base1);
  float rs0 = e00 + e01 + e10 + e11;
  float rs1 = f00 + f01 + f10 + f11;
  rs0 += __shfl_xor_sync(0xffffffffu, rs0, 1);
  rs0 += __shfl_xor_sync(0xffffffffu, rs0, 2);
  rs1 += __shfl_xor_sync(0xffffffffu, rs1, 1);
  rs1 += __shfl_xor_sync(0xffffffffu, rs1, 2);
  st.l0 = st.l0 * corr0 + rs0;
  st.l1 = st.l1 * corr1 + rs1;
  st.m0 = mn0;
  st.m1 = mn1;
#pragma unroll
  for (int n = 0; n < D / 8; ++n) {
    o[n][0] *= corr0; o[n][1] *= corr0;
    o[n][2] *= corr1; o[n][3] *= corr1;
  }
  // C fragments of two adjacent 8-key tiles form the A fragment of one 16-key step
  p0 = pack_bf16x2(e00, e01);
  p1 = pack_bf16x2(f00, f01);
  p2 = pack_bf16x2(e10, e11);
  p3 = pack_bf16x2(f10, f11);
}

// ------------------------------------------------------------------------------------------
// Decode
// ------------------------------------------------------------------------------------------
constexpr int DEC_WARPS = 4;
constexpr int DEC_STAGES = 3;  // 50 KB (D=64) / 100 KB (D=128) per CTA -> 4 / 2 CTAs per SM

template <int D>
__global__ void __launch_bounds__(DEC_WARPS * 32)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q,         // [B, Hq, D]
                    const __nv_bfloat16* __restrict__ k_cache,   // [num_blocks, Hkv, 16, D]
                    const __nv_bfloat16* __restrict__ v_cache,
                    const int* __restrict__ block_tables,        // [B, max_blocks]
                    const int* __restrict__ seq_lens,            // [B]
                    __nv_bfloat16* __restrict__ out,             // [B, Hq, D]
                    float* __restrict__ part_o,                  // [B, Hq, S, D]   (S > 1)
                    float* __restrict__ part_ml,                 // [B, Hq, S, 2]
                    int Hq, int Hkv, int max_blocks, int num_blocks, int num_splits, float scale,
                    int* status) {
  constexpr int CH = D / 8;                 // 16-byte chunks per row
  constexpr int TILE_BYTES = KV_BLOCK * D * 2;
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = Hq / Hkv;
  const int L = seq_lens[b];
  const int n_chunks = (L + KV_BLOCK - 1) / KV_BLOCK;
  const int per = (n_chunks + num_splits - 1) / num_splits;
  const int c_begin = split * per;
  const int c_end = min(n_chunks, c_begin + per);

  // shared memory: Q tile [16][D] then per warp DEC_STAGES x (K tile, V tile)
  const uint32_t q_smem = smem_u32(smem);
  const uint32_t kv_smem = q_smem + 16 * D * 2 + warp * (DEC_STAGES * 2 * TILE_BYTES);

  // stage Q (rows >= G zero)
  for (int i = threadIdx.x; i < 16 * CH; i += blockDim.x) {
    const int r = i / CH, c = i % CH;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < G) v = *reinterpret_cast<const uint4*>(q + ((long long)b * Hq + kvh * G + r) * D + c * 8);
    *reinterpret_cast<uint4*>(smem + swz<D>(r, c)) = v;
  }
  __syncthreads();
  uint32_t qf[D / 16][4];
  {
    const int mat = lane >> 3, r = lane & 7;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks)
      ldsm_x4(q_smem + swz<D>((mat & 1) * 8 + r, 2 * ks + (mat >> 1)), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
  }

  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
  RowState st = {-INFINITY, -INFINITY, 0.f, 0.f};
  const float scale_log2 = scale * 1.4426950408889634f;

  auto issue = [&](int chunk, int stage) {
    if (chunk < c_end) {
      int blk = block_tables[(long long)b * max_blocks + chunk];
      if (blk < 0 || blk >= num_blocks) { set_status(status, ST_BAD_INDEX); blk = 0; }
      const __nv_bfloat16* ksrc = k_cache + ((long long)blk * Hkv + kvh) * KV_BLOCK * D;
      const __nv_bfloat16* vsrc = v_cache + ((long long)blk * Hkv + kvh) * KV_BLOCK * D;
      const uint32_t ks = kv_smem + stage * 2 * TILE_BYTES, vs = ks + TILE_BYTES;
#pragma unroll
      for (int i = lane; i < KV_BLOCK * CH; i += 32) {
        const int r = i / CH, c = i % CH;
        cp_async16(ks + swz<D>(r, c), ksrc + r * D + c * 8);
        cp_async16(vs + swz<D>(r, c), vsrc + r * D + c * 8);
      }
    }
    cp_async_commit();
  };

  int my = c_begin + warp;
#pragma unroll
  for (int s = 0; s < DEC_STAGES - 1; ++s) issue(my + s * DEC_WARPS, s);
  int stage = 0;
  for (int chunk = my; chunk < c_end; chunk += DEC_WARPS) {
    issue(chunk + (DEC_STAGES - 1) * DEC_WARPS, (stage + DEC_STAGES - 1) % DEC_STAGES);
    cp_async_wait<DEC_STAGES - 1>();
    __syncwarp();
    const uint32_t ks = kv_smem + stage * 2 * TILE_BYTES, vs = ks + TILE_BYTES;
    float s0[4] = {0, 0, 0, 0}, s1[4] = {0, 0, 0, 0};
    qk_16x16<D>(s0, s1, qf, ks, 0, lane);
    const int tok0 = chunk * KV_BLOCK + 2 * (lane & 3);
    if (tok0 >= L) { s0[0] = s0[2] = -INFINITY; }
    if (tok0 + 1 >= L) { s0[1] = s0[3] = -INFINITY; }
    if (tok0 + 8 >= L) { s1[0] = s1[2] = -INFINITY; }
    if (tok0 + 9 >= L) { s1[1] = s1[3] = -INFINITY; }
    uint32_t p0, p1, p2, p3;
    softmax_update<D>(s0, s1, st, o, scale_log2, p0, p1, p2, p3);
    pv_16x16<D>(o, p0, p1, p2, p3, vs, 0, lane);
    __syncwarp();
    stage = (stage + 1) % DEC_STAGES;
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- merge the warps through shared memory (re-using the KV ring) ----
  float* mo = reinterpret_cast<float*>(smem + 16 * D * 2);          // [DEC_WARPS][8][D]
  float* mml = mo + DEC_WARPS * 8 * D;                              // [DEC_WARPS][8][2]
  const int g = lane >> 2, t = lane & 3;
  if (g < 8) {
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      mo[(warp * 8 + g) * D + n * 8 + 2 * t] = o[n][0];
      mo[(warp * 8 + g) * D + n * 8 + 2 * t + 1] = o[n][1];
    }
    if (t == 0) { mml[(warp * 8 + g) * 2] = st.m0; mml[(warp * 8 + g) * 2 + 1] = st.l0; }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int r = i / D, d = i % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, mml[(w * 8 + r) * 2]);
    float acc = 0.f, l = 0.f;
    if (M != -INFINITY) {
#pragma unroll
      for (int w = 0; w < DEC_WARPS; ++w) {
        const float e = exp2f(mml[(w * 8 + r) * 2] - M);
        acc += e * mo[(w * 8 + r) * D + d];
        l += e * mml[(w * 8 + r) * 2 + 1];
      }
    }
    const int h = kvh * G + r;
    if (num_splits == 1) {
      out[((long long)b * Hq + h) * D + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
    } else {
      const long long pi = ((long long)b * Hq + h) * num_splits + split;
      part_o[pi * D + d] = acc;
      if (d == 0) { part_ml[pi * 2] = M; part_ml[pi * 2 + 1] = l; }
    }
  }
}

// ------------------------------------------------------------------------------------------
// Decode, TMA variant (default): every 16-token block of one KV head is a contiguous [16, D]
// tile, fetched with ONE tile copy per 128 bytes of row (1 for D=64, 2 for D=128) instead of 128
// sixteen-byte requests. The 128-byte swizzle of the copy is exactly the XOR layout ldmatrix
// needs. Each warp owns a ring of 3-4 (K,V) tiles with one mbarrier per stage; an
// out-of-range block id lands on an out-of-bounds coordinate, which TMA fills with zeros.
// ------------------------------------------------------------------------------------------
template <int D>
__host__ __device__ constexpr int dec_tma_stages() { return 3; }   // 52 KB (D=64: 4 CTAs/SM) or 103 KB (D=128: 2 CTAs/SM)

// 16-byte chunk c of row r inside a [16, D] tile loaded as D/64 swizzled [16][128 B] half tiles
template <int D>
__device__ __forceinline__ uint32_t swz_tma(int r, int c) {
  return (uint32_t)((c >> 3) * (KV_BLOCK * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4));
}

template <int D>
__global__ void __launch_bounds__(DEC_WARPS * 32)
paged_decode_tma_kernel(const __nv_bfloat16* __restrict__ q, const __grid_constant__ CUtensorMap k_map,
                        const __grid_constant__ CUtensorMap v_map, const int* __restrict__ block_tables,
                        const int* __restrict__ seq_lens, __nv_bfloat16* __restrict__ out,
                        float* __restrict__ part_o, float* __restrict__ part_ml, int Hq, int Hkv, int max_blocks,
                        int num_blocks, int num_splits, float scale, int* status) {
  constexpr int CH = D / 8;
  constexpr int TILE_BYTES = KV_BLOCK * D * 2;
  constexpr int ST = dec_tma_stages<D>();
  extern __shared__ __align__(128) uint8_t smem[];   // the ring is aligned to 1024 bytes by hand below
  __shared__ __align__(8) uint64_t bars[DEC_WARPS][ST];
  __shared__ int abort_flag;
  pdl_launch_dependents();
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = Hq / Hkv;
  // layout: [ring: DEC_WARPS x ST x (K tile, V tile)] (1024-byte aligned) then the Q tile
  const uint32_t ring0 = (smem_u32(smem) + 1023u) & ~1023u;
  uint8_t* ring_ptr = smem + (ring0 - smem_u32(smem));
  const uint32_t kv_smem = ring0 + warp * (ST * 2 * TILE_BYTES);
  uint8_t* q_ptr = ring_ptr + DEC_WARPS * ST * 2 * TILE_BYTES;
  const uint32_t q_smem = smem_u32(q_ptr);
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int w = 0; w < DEC_WARPS; ++w)
      for (int s2 = 0; s2 < ST; ++s2) mbar_init(smem_u32(&bars[w][s2]), 1);
    fence_mbar_init();
  }
  pdl_wait();
  const int L = seq_lens[b];
  const int n_chunks = (L + KV_BLOCK - 1) / KV_BLOCK;
  const int per = (n_chunks + num_splits - 1) / num_splits;
  const int c_begin = split * per;
  const int c_end = min(n_chunks, c_begin + per);
  for (int i = threadIdx.x; i < 16 * CH; i += blockDim.x) {
    const int r = i / CH, c = i % CH;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < G) v = *reinterpret_cast<const uint4*>(q + ((long long)b * Hq + kvh * G + r) * D + c * 8);
    *reinterpret_cast<uint4*>(q_ptr + swz<D>(r, c)) = v;
  }
  __syncthreads();
  uint32_t qf[D / 16][4];
  {
    const int mat = lane >> 3, r = lane & 7;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks)
      ldsm_x4(q_smem + swz<D>((mat & 1) * 8 + r, 2 * ks + (mat >> 1)), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
  }
  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
  RowState st = {-INFINITY, -INFINITY, 0.f, 0.f};
  const float scale_log2 = scale * 1.4426950408889634f;
  volatile int* abortp = &abort_flag;

  const int first = c_begin + warp;
  const int n_my = first < c_end ? (c_end - first + DEC_WARPS - 1) / DEC_WARPS : 0;
  // Block ids of this warp's chunks are fetched 32 at a time (lane j holds chunk round*32+j) so the
  // table lookup is off the critical path of every copy.
  const int* bt_row = block_tables + (long long)b * max_blocks;
  auto load_ids = [&](int round) {
    const int j = round * 32 + lane;
    return j < n_my ? __ldg(bt_row + first + j * DEC_WARPS) : 0;
  };
  int ids_round = 0, ids = load_ids(0), ids_next = load_ids(1);
  auto blk_of = [&](int i) {   // all lanes, i uniform and non-decreasing
    if ((i >> 5) > ids_round) { ids = ids_next; ids_round = i >> 5; ids_next = load_ids(ids_round + 1); }
    return __shfl_sync(0xffffffffu, ids, i & 31);
  };
  auto issue = [&](int i, int blk) {   // lane 0 only
    const int stage = i % ST;
    if (blk < 0 || blk >= num_blocks) { set_status(status, ST_BAD_INDEX); blk = num_blocks; }  // OOB -> zeros
    const int y = (blk * Hkv + kvh) * KV_BLOCK;
    const uint32_t bar = smem_u32(&bars[warp][stage]);
    const uint32_t ks = kv_smem + stage * 2 * TILE_BYTES, vs = ks + TILE_BYTES;
    mbar_expect_tx(bar, 2 * TILE_BYTES);
#pragma unroll
    for (int hx = 0; hx < D / 64; ++hx) {
      tma_load_2d(ks + hx * (KV_BLOCK * 128), &k_map, bar, hx * 64, y);
      tma_load_2d(vs + hx * (KV_BLOCK * 128), &v_map, bar, hx * 64, y);
    }
  };
  int issued = 0;
  for (; issued < ST - 1 && issued < n_my; ++issued) {
    const int blk = blk_of(issued);
    if (lane == 0) issue(issued, blk);
  }
  bool ok = true;
  const int mat = lane >> 3, rr = lane & 7;
  for (int i = 0; i < n_my; ++i) {
    if (issued < n_my) {
      const int blk = blk_of(issued);
      if (lane == 0) issue(issued, blk);
      ++issued;
    }
    const int stage = i % ST;
    ok = mbar_wait_bounded(smem_u32(&bars[warp][stage]), (uint32_t)((i / ST) & 1), abortp, status, ST_TIMEOUT_SMEM_FULL);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;
    const uint32_t ks = kv_smem + stage * 2 * TILE_BYTES, vs = ks + TILE_BYTES;
    float s0[4] = {0, 0, 0, 0}, s1[4] = {0, 0, 0, 0};
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t b0, b1, b2, b3;
      ldsm_x4(ks + swz_tma<D>((mat >> 1) * 8 + rr, 2 * kk + (mat & 1)), b0, b1, b2, b3);
      mma_16816(s0, qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b0, b1);
      mma_16816(s1, qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b2, b3);
    }
    const int tok0 = (first + i * DEC_WARPS) * KV_BLOCK + 2 * (lane & 3);
    if (tok0 >= L) { s0[0] = s0[2] = -INFINITY; }
    if (tok0 + 1 >= L) { s0[1] = s0[3] = -INFINITY; }
    if (tok0 + 8 >= L) { s1[0] = s1[2] = -INFINITY; }
    if (tok0 + 9 >= L) { s1[1] = s1[3] = -INFINITY; }
    uint32_t p0, p1, p2, p3;
    softmax_update<D>(s0, s1, st, o, scale_log2, p0, p1, p2, p3);
#pragma unroll
    for (int dp = 0; dp < D / 16; ++dp) {
      uint32_t b0, b1, b2, b3;
      ldsm_x4_t(vs + swz_tma<D>((mat & 1) * 8 + rr, 2 * dp + (mat >> 1)), b0, b1, b2, b3);
      mma_16816(o[2 * dp], p0, p1, p2, p3, b0, b1);
      mma_16816(o[2 * dp + 1], p0, p1, p2, p3, b2, b3);
    }
    __syncwarp();   // every lane is done with this stage before lane 0 refills it
  }
  if (!ok && lane == 0) {
    // drain: wait (bounded) for copies already issued so none lands after the CTA has exited
    for (int j = max(0, issued - ST); j < issued; ++j) {   // the latest phase of every stage
      const uint64_t t0 = globaltimer_ns();
      while (!mbar_try_wait(smem_u32(&bars[warp][j % ST]), (uint32_t)((j / ST) & 1)))
        if (globaltimer_ns() - t0 > 50000000ull) break;
    }
  }
  __syncthreads();

  float* mo = reinterpret_cast<float*>(ring_ptr);                   // [DEC_WARPS][8][D]
  float* mml = mo + DEC_WARPS * 8 * D;                              // [DEC_WARPS][8][2]
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int n = 0; n < D / 8; ++n) {
    mo[(warp * 8 + g) * D + n * 8 + 2 * t] = o[n][0];
    mo[(warp * 8 + g) * D + n * 8 + 2 * t + 1] = o[n][1];
  }
  if (t == 0) { mml[(warp * 8 + g) * 2] = st.m0; mml[(warp * 8 + g) * 2 + 1] = st.l0; }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int r = i / D, d = i % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, mml[(w * 8 + r) * 2]);
    float acc = 0.f, l = 0.f;
    if (M != -INFINITY) {
#pragma unroll
      for (int w = 0; w < DEC_WARPS; ++w) {
        const float e = exp2f(mml[(w * 8 + r) * 2] - M);
        acc += e * mo[(w * 8 + r) * D + d];
        l += e * mml[(w * 8 + r) * 2 + 1];
      }
    }
    const int h = kvh * G + r;
    if (num_splits == 1) {
      out[((long long)b * Hq + h) * D + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
    } else {
      const long long pi = ((long long)b * Hq + h) * num_splits + split;
      part_o[pi * D + d] = acc;
      if (d == 0) { part_ml[pi * 2] = M; part_ml[pi * 2 + 1] = l; }
    }
  }
}

template <int D>
__global__ void decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    __nv_bfloat16* __restrict__ out, int num_splits) {
  pdl_launch_dependents();
  pdl_wait();
  const long long bh = blockIdx.x;
  const int d = threadIdx.x;
  if (d >= D) return;
  float M = -INFINITY;
  for (int s = 0; s < num_splits; ++s) M = fmaxf(M, part_ml[(bh * num_splits + s) * 2]);
  float acc = 0.f, l = 0.f;
  if (M != -INFINITY) {
    for (int s = 0; s < num_splits; ++s) {
      const float e = exp2f(part_ml[(bh * num_splits + s) * 2] - M);
      acc += e * part_o[(bh * num_splits + s) * D + d];
      l += e * part_ml[(bh * num_splits + s) * 2 + 1];
    }
  }
  out[bh * D + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
}

// ------------------------------------------------------------------------------------------
// Prefill (varlen, causal, prefix-aware, optional sliding window)
// ------------------------------------------------------------------------------------------
constexpr int PF_WARPS = 4;
constexpr int PF_BM = 64;
constexpr int PF_BN = 64;

template <int D>
__global__ void __launch_bounds__(PF_WARPS * 32)
paged_prefill_kernel(const __nv_bfloat16* __restrict__ q,        // [T, Hq, D] packed new tokens
                     const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                     const int* __restrict__ block_tables,       // [B, max_blocks]
                     const int* __restrict__ cu_q,               // [B+1] offsets of new tokens
                     const int* __restrict__ seq_lens,           // [B] total context (prefix + new)
                     __nv_bfloat16* __restrict__ out,            // [T, Hq, D]
                     float* __restrict__ lse,                    // [T, Hq] natural-log LSE or null
                     int Hq, int Hkv, int max_blocks, int num_blocks, float scale, int window,
                     int* status) {
  constexpr int CH = D / 8;
  constexpr int KTILE_BYTES = PF_BN * D * 2;
  extern __shared__ __align__(128) uint8_t smem[];
  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q_begin = cu_q[b], q_end = cu_q[b + 1];
  const int n_new = q_end - q_begin;
  if (qt * PF_BM >= n_new) return;
  const int L = seq_lens[b];
  const int prefix = L - n_new;                 // tokens already cached before this call
  const int kvh = h / (Hq / Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t q_smem = smem_u32(smem);
  const uint32_t k_smem0 = q_smem + PF_BM * D * 2;          // 2 stages of K then 2 stages of V
  const uint32_t v_smem0 = k_smem0 + 2 * KTILE_BYTES;

  for (int i = threadIdx.x; i < PF_BM * CH; i += blockDim.x) {
    const int r = i / CH, c = i % CH;
    const int tq = qt * PF_BM + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (tq < n_new) v = *reinterpret_cast<const uint4*>(q + ((long long)(q_begin + tq) * Hq + h) * D + c * 8);
    *reinterpret_cast<uint4*>(smem + swz<D>(r, c)) = v;
  }
  __syncthreads();
  uint32_t qf[D / 16][4];
  {
    const int mat = lane >> 3, r = lane & 7;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks)
      ldsm_x4(q_smem + swz<D>(warp * 16 + (mat & 1) * 8 + r, 2 * ks + (mat >> 1)), qf[ks][0], qf[ks][1], qf[ks][2],
              qf[ks][3]);
  }

  // absolute positions of this thread's two query rows
  const int g = lane >> 2, t4 = lane & 3;
  const int row0 = qt * PF_BM + warp * 16 + g, row1 = row0 + 8;
  const int pos0 = prefix + row0, pos1 = prefix + row1;
  // keys needed by this CTA: [k_lo, k_hi)
  const int last_q = min(n_new, (qt + 1) * PF_BM) - 1;
  const int k_hi = min(L, prefix + last_q + 1);
  int k_lo = 0;
  if (window > 0) k_lo = max(0, prefix + qt * PF_BM - window + 1);
  const int tile_lo = k_lo / PF_BN, tile_hi = (k_hi + PF_BN - 1) / PF_BN;

  auto issue = [&](int tile, int stage) {
    if (tile < tile_hi) {
      const uint32_t ks = k_smem0 + stage * KTILE_BYTES, vs = v_smem0 + stage * KTILE_BYTES;
      for (int i = threadIdx.x; i < PF_BN * CH; i += blockDim.x) {
        const int r = i / CH, c = i % CH;
        const int key = tile * PF_BN + r;
        if (key < L) {
          int blk = block_tables[(long long)b * max_blocks + key / KV_BLOCK];
          if (blk < 0 || blk >= num_blocks) { set_status(status, ST_BAD_INDEX); blk = 0; }
          const long long off = (((long long)blk * Hkv + kvh) * KV_BLOCK + (key % KV_BLOCK)) * D + c * 8;
          cp_async16(ks + swz<D>(r, c), k_cache + off);
          cp_async16(vs + swz<D>(r, c), v_cache + off);
        } else {
          // rows past the sequence end are masked below, but V must not hold NaN garbage
          *reinterpret_cast<uint4*>(smem + (vs - q_smem) + swz<D>(r, c)) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(smem + (ks - q_smem) + swz<D>(r, c)) = make_uint4(0, 0, 0, 0);
        }
      }
    }
    cp_async_commit();
  };

  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
  RowState st = {-INFINITY, -INFINITY, 0.f, 0.f};
  const float scale_log2 = scale * 1.4426950408889634f;

  issue(tile_lo, 0);
  int stage = 0;
  for (int tile = tile_lo; tile < tile_hi; ++tile) {
    issue(tile + 1, stage ^ 1);
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t ks = k_smem0 + stage * KTILE_BYTES, vs = v_smem0 + stage * KTILE_BYTES;
#pragma unroll
    for (int kk = 0; kk < PF_BN / 16; ++kk) {
      const int key_base = tile * PF_BN + kk * 16;
      // skip 16-key steps that are entirely in this warp's causal future
      if (key_base > prefix + qt * PF_BM + warp * 16 + 15) continue;
      float s0[4] = {0, 0, 0, 0}, s1[4] = {0, 0, 0, 0};
      qk_16x16<D>(s0, s1, qf, ks, kk * 16, lane);
      const int c0 = key_base + 2 * t4;
      auto dead = [&](int key, int pos) {
        return key > pos || key >= L || (window > 0 && key <= pos - window);
      };
      if (dead(c0, pos0)) s0[0] = -INFINITY;
      if (dead(c0 + 1, pos0)) s0[1] = -INFINITY;
      if (dead(c0, pos1)) s0[2] = -INFINITY;
      if (dead(c0 + 1, pos1)) s0[3] = -INFINITY;
      if (dead(c0 + 8, pos0)) s1[0] = -INFINITY;
      if (dead(c0 + 9, pos0)) s1[1] = -INFINITY;
      if (dead(c0 + 8, pos1)) s1[2] = -INFINITY;
      if (dead(c0 + 9, pos1)) s1[3] = -INFINITY;
      uint32_t p0, p1, p2, p3;
      softmax_update<D>(s0, s1, st, o, scale_log2, p0, p1, p2, p3);
      pv_16x16<D>(o, p0, p1, p2, p3, vs, kk * 16, lane);
    }
    __syncthreads();
    stage ^= 1;
  }
  cp_async_wait<0>();

  const float inv0 = st.l0 > 0.f ? 1.f / st.l0 : 0.f;
  const float inv1 = st.l1 > 0.f ? 1.f / st.l1 : 0.f;
  if (row0 < n_new) {
    __nv_bfloat16* dst = out + ((long long)(q_begin + row0) * Hq + h) * D;
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
      *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * t4) = pack_bf16x2(o[n][0] * inv0, o[n][1] * inv0);
    if (lse != nullptr && t4 == 0)
      lse[(long long)(q_begin + row0) * Hq + h] = (st.m0 + log2f(st.l0)) * 0.6931471805599453f;
  }
  if (row1 < n_new) {
    __nv_bfloat16* dst = out + ((long long)(q_begin + row1) * Hq + h) * D;
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
      *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * t4) = pack_bf16x2(o[n][2] * inv1, o[n][3] * inv1);
    if (lse != nullptr && t4 == 0)
      lse[(long long)(q_begin + row1) * Hq + h] = (st.m1 + log2f(st.l1)) * 0.6931471805599453f;
  }
}

template <int D>
constexpr int decode_smem_bytes() {
  return 16 * D * 2 + DEC_WARPS * DEC_STAGES * 2 * KV_BLOCK * D * 2;
}
template <int D>
constexpr int decode_tma_smem_bytes() {
  return 1024 + DEC_WARPS * dec_tma_stages<D>() * 2 * KV_BLOCK * D * 2 + 16 * D * 2;
}
template <int D>
constexpr int prefill_smem_bytes() {
  return PF_BM * D * 2 + 4 * PF_BN * D * 2;
}

}  // namespace rb

using namespace rb;

extern "C" void rb_attn_set_pdl(int on) { rb::pdl_enabled() = on != 0; }

// Function attributes (the dynamic shared-memory opt-in) belong to a device, so the "already set" flags of the
// launchers below are kept per device: a process that drives several GPUs sets them on each.
#define RB_MAX_DEVICES 64
static int current_device_index() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= RB_MAX_DEVICES) return -1;
  return dev;
}

// Scratch needed by rb_paged_decode when num_splits > 1, in floats.
extern "C" long long rb_paged_decode_workspace_floats(int B, int Hq, int D, int num_splits) {
  if (num_splits <= 1) return 0;
  return (long long)B * Hq * num_splits * (D + 2);
}

extern "C" int rb_paged_decode(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                               const int* seq_lens, void* out, float* workspace, int B, int Hq, int Hkv, int D,
                               int max_blocks, int num_blocks, int block_size, int num_splits, float scale,
                               int* status, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (block_size != KV_BLOCK || Hq % Hkv != 0 || Hq / Hkv > 8 || num_splits < 1) return -1;
  if (num_splits > 1 && workspace == nullptr) return -1;
  float* part_o = workspace;
  float* part_ml = workspace ? workspace + (long long)B * Hq * num_splits * D : nullptr;
  dim3 grid(num_splits, Hkv, B);
  static const bool use_cpasync = getenv("RB_DECODE_CPASYNC") != nullptr;
  if (!use_cpasync) {
    CUtensorMap kmap, vmap;
    const unsigned long long rows = (unsigned long long)num_blocks * Hkv * KV_BLOCK;
    if (tma_map_2d_bf16(&kmap, k_cache, rows, D, D, KV_BLOCK) != 0) return -20;
    if (tma_map_2d_bf16(&vmap, v_cache, rows, D, D, KV_BLOCK) != 0) return -21;
#define LAUNCH_DEC_TMA(DD)                                                                                    \
  do {                                                                                                        \
    static bool attr[RB_MAX_DEVICES] = {};   /* the opt-in above 48 KB is a per-device function attribute */  \
    const int dev_ = current_device_index();                                                                  \
    if (dev_ < 0) return -10;                                                                                 \
    if (!attr[dev_]) {                                                                                        \
      if (cudaFuncSetAttribute(paged_decode_tma_kernel<DD>, cudaFuncAttributeMaxDynamicSharedMemorySize,      \
                               decode_tma_smem_bytes<DD>()) != cudaSuccess) return -10;                       \
      attr[dev_] = true;                                                                                      \
    }                                                                                                         \
    launch_kernel(paged_decode_tma_kernel<DD>, grid, dim3(DEC_WARPS * 32), decode_tma_smem_bytes<DD>(), stream, \
        (const __nv_bfloat16*)q, kmap, vmap, block_tables, seq_lens, (__nv_bfloat16*)out, part_o, part_ml, Hq, \
        Hkv, max_blocks, num_blocks, num_splits, scale, status);                                              \
    if (num_splits > 1)                                                                                       \
      launch_kernel(decode_merge_kernel<DD>, dim3(B * Hq), dim3(DD), 0, stream, (const float*)part_o,         \
                    (const float*)part_ml, (__nv_bfloat16*)out, num_splits);                                  \
  } while (0)
    if (D == 64) LAUNCH_DEC_TMA(64);
    else if (D == 128) LAUNCH_DEC_TMA(128);
    else return -1;
#undef LAUNCH_DEC_TMA
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
  }
#define LAUNCH_DEC(DD)                                                                                        \
  do {                                                                                                        \
    static bool attr[RB_MAX_DEVICES] = {};                                                                    \
    const int dev_ = current_device_index();                                                                  \
    if (dev_ < 0) return -10;                                                                                 \
    if (!attr[dev_]) {                                                                                        \
      if (cudaFuncSetAttribute(paged_decode_kernel<DD>, cudaFuncAttributeMaxDynamicSharedMemorySize,          \
                               decode_smem_bytes<DD>()) != cudaSuccess) return -10;                           \
      attr[dev_] = true;                                                                                      \
    }                                                                                                         \
    launch_kernel(paged_decode_kernel<DD>, grid, dim3(DEC_WARPS * 32), decode_smem_bytes<DD>(), stream,        \
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, block_tables,  \
        seq_lens, (__nv_bfloat16*)out, part_o, part_ml, Hq, Hkv, max_blocks, num_blocks, num_splits, scale,   \
        status);                                                                                              \
    if (num_splits > 1)                                                                                       \
      launch_kernel(decode_merge_kernel<DD>, dim3(B * Hq), dim3(DD), 0, stream, (const float*)part_o,         \
                    (const float*)part_ml, (__nv_bfloat16*)out, num_splits);                                  \
  } while (0)
  if (D == 64) LAUNCH_DEC(64);
  else if (D == 128) LAUNCH_DEC(128);
  else return -1;
#undef LAUNCH_DEC
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int rb_paged_prefill(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                                const int* cu_q, const int* seq_lens, void* out, float* lse, int B, int max_new,
                                int Hq, int Hkv, int D, int max_blocks, int num_blocks, int block_size, float scale,
                                int window, int* status, cudaStream_t stream) {
  if (B <= 0 || max_new <= 0) return 0;
  if (block_size != KV_BLOCK || Hq % Hkv != 0) return -1;
  dim3 grid((max_new + PF_BM - 1) / PF_BM, Hq, B);
#define LAUNCH_PF(DD)                                                                                         \
  do {                                                                                                        \
    static bool attr[RB_MAX_DEVICES] = {};                                                                    \
    const int dev_ = current_device_index();                                                                  \
    if (dev_ < 0) return -10;                                                                                 \
    if (!attr[dev_]) {                                                                                        \
      if (cudaFuncSetAttribute(paged_prefill_kernel<DD>, cudaFuncAttributeMaxDynamicSharedMemorySize,         \
                               prefill_smem_bytes<DD>()) != cudaSuccess) return -10;                          \
      attr[dev_] = true;                                                                                      \
    }                                                                                                         \
    paged_prefill_kernel<DD><<<grid, PF_WARPS * 32, prefill_smem_bytes<DD>(), stream>>>(                       \
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, block_tables,  \
        cu_q, seq_lens, (__nv_bfloat16*)out, lse, Hq, Hkv, max_blocks, num_blocks, scale, window, status);    \
  } while (0)
  if (D == 64) LAUNCH_PF(64);
  else if (D == 128) LAUNCH_PF(128);
  else return -1;
#undef LAUNCH_PF
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// ------------------------------------------------------------------------------------------
// Allocation-free variant (see attn_noalloc.h for the contract and for who needs it).
// ------------------------------------------------------------------------------------------
#include "attn_noalloc.h"

#include <mutex>

// Per-split partial outputs and (max, sum) pairs. In host code this name is only a handle for
// the runtime, not a device address: the address is fetched with cudaGetSymbolAddress below.
static __device__ __align__(256) float rb_decode_noalloc_scratch[RB_DECODE_NOALLOC_MAX_FLOATS];

namespace {
constexpr int kMaxDevices = RB_MAX_DEVICES;
float* g_noalloc_ptr[kMaxDevices] = {};
std::mutex g_noalloc_mutex;

// Device address of the scratch array on the current device, looked up once per device.
int noalloc_scratch_for_current_device(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return RB_NOALLOC_SYMBOL_LOOKUP_FAILED;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_ptr[dev] == nullptr) {
    float* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), rb_decode_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) return RB_NOALLOC_SYMBOL_LOOKUP_FAILED;
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return 0;
}
}  // namespace

extern "C" long long rb_paged_decode_noalloc_required_floats(int B, int Hq, int D, int num_splits) {
  // one split writes the output directly: nothing of the array is touched, whatever the batch
  if (B <= 0 || Hq <= 0 || D <= 0 || num_splits <= 1) return 0;
  return (long long)B * Hq * num_splits * (D + 2);
}

extern "C" int rb_paged_decode_noalloc(const void* q, const void* k_cache, const void* v_cache,
                                       const int* block_tables, const int* seq_lens, void* out, int B, int Hq,
                                       int Hkv, int D, int max_blocks, int num_blocks, int block_size, int num_splits,
                                       float scale, int* status, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (num_splits < 1) return -1;
  if (rb_paged_decode_noalloc_required_floats(B, Hq, D, num_splits) > (long long)RB_DECODE_NOALLOC_MAX_FLOATS)
    return RB_NOALLOC_TOO_LARGE;
  float* scratch = nullptr;
  if (num_splits > 1) {   // a single split needs no workspace, so no lookup either
    const int rc = noalloc_scratch_for_current_device(&scratch);
    if (rc != 0) return rc;
  }
  // Same kernels and launch logic as the regular entry point, with the library's own workspace.
  return rb_paged_decode(q, k_cache, v_cache, block_tables, seq_lens, out, scratch, B, Hq, Hkv, D, max_blocks,
                         num_blocks, block_size, num_splits, scale, status, stream);
}
