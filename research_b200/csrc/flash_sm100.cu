// Flash attention for sm_100a on the 5th-generation tensor cores.
//
// Forward: one CTA owns 128 query rows of one head. S = Q K^T and O += P V are tcgen05.mma
// instructions issued by one thread; S (two buffers) and O live in tensor memory, Q/K/V tiles are
// brought into 128-byte-swizzled shared memory by TMA, P goes back to shared memory as the A operand
// of the second product. Warp roles: warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2-9
// softmax (two threads per query row, each reading half of it from TMEM with tcgen05.ld). The running maximum is only
// refreshed when it grew by more than 2^8, so the O accumulator is rescaled rarely.
//
// Inputs are packed variable-length batches (`cu_seqlens`), grouped-query heads, causal and
// sliding-window masks; K/V come either from dense [T, Hkv, D] tensors (training) or from the paged
// cache [num_blocks, Hkv, 16, D] through a block table (prefill with a cached prefix).
//
// Replaces F.scaled_dot_product_attention / FlexAttention in the reference
// (rollouts/inference/attention/flex_backend.py:144-185) and the Hopper-only varlen flash kernel of
// dev/speedrun/single-file.py:932-943.
//
// Every wait is bounded; on a timeout the kernel records a status code, drains its copies, frees
// tensor memory and returns.
#include "common.cuh"
#include "tma_host.h"

#include <math.h>
#include <stdlib.h>

namespace rb {

constexpr int FA_BM = 128;        // query rows per CTA
constexpr int FA_BN = 128;        // keys per iteration
constexpr int FA_THREADS = 320;   // 10 warps: TMA, MMA, two softmax warpgroups
constexpr int FA_KV_SLOTS = 3;    // ring of K/V tiles in consumption order: K0 K1 V0 K2 V1 K3 V2 ...
constexpr int FA_TMEM_COLS = 512;
constexpr float FA_RESCALE_THRESHOLD = 8.f;   // log2 units

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Wait for the single-thread producer / MMA roles. `mbarrier.try_wait` with a suspend-time hint parks the thread in
// hardware until the phase completes or the hint runs out: the waiter takes no issue slots from the softmax warps
// on its scheduler (what a plain poll loop did) and wakes as soon as the barrier flips (what a poll + nanosleep
// loop did not: at short sequences every hand-off on the critical path paid a sleep quantum).
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return done != 0;
}
__device__ __forceinline__ bool mbar_wait_backoff(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                                  int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait_hint(bar, parity, 2000u)) return true;
    if ((++spins & 0x3f) == 0) {
      if (*abort_flag != 0) return false;
      if (globaltimer_ns() - t0 > RB_WAIT_BUDGET_NS) {
        *abort_flag = 1;
        set_status(status, code);
        return false;
      }
    }
  }
}

struct FlashFwdParams {
  CUtensorMap q_map;   // [Tq, Hq*D], box 64 x 128
  CUtensorMap k_map;   // dense: [Tk, Hkv*D], box 64 x 128; paged: [num_blocks*Hkv*16, D], box 64 x 16
  CUtensorMap v_map;
  __nv_bfloat16* out;  // [Tq, Hq, D]
  float* lse;          // [Hq, Tq] natural-log sum-exp of the scaled scores
  const int* cu_q;     // [B+1]
  const int* cu_k;     // [B+1] (dense)
  const int* seq_lens; // [B] total keys per sequence (paged)
  const int* block_tables;  // [B, max_blocks] (paged)
  int max_blocks, num_blocks;
  int Hq, Hkv, Tq;
  int causal, window, paged;
  float scale_log2;
  int* status;
};

template <int D>
struct FlashCfg {
  static constexpr int kTileBytes = FA_BN * D * 2;          // one K or V tile (and the Q tile)
  static constexpr int kPBytes = FA_BM * FA_BN * 2;
  static constexpr int kSmemBytes = 1024 + kTileBytes + FA_KV_SLOTS * kTileBytes + 2 * kPBytes;
};

template <int D>
__global__ void __launch_bounds__(FA_THREADS, 1) flash_fwd_kernel(const __grid_constant__ FlashFwdParams p) {
  using Cfg = FlashCfg<D>;
  constexpr int DCH = D / 64;                    // 64-column chunks of the head dimension
  constexpr int CHUNK_BYTES = FA_BN * 128;       // 128 rows x 128 B
  extern __shared__ __align__(128) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t q_full, kv_full[FA_KV_SLOTS], kv_empty[FA_KV_SLOTS];
  __shared__ __align__(8) uint64_t s_full[2], s_empty[2], p_full[2], p_empty[2], o_done, xch_bar[4];
  __shared__ float xch[2][2][FA_BM];
  __shared__ uint32_t tmem_base_smem;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, h = blockIdx.y;
  const int q_tile = gridDim.x - 1 - blockIdx.x;           // long (late) tiles first
  const int q_begin = p.cu_q[b];
  const int q_len = p.cu_q[b + 1] - q_begin;
  const int q0 = q_tile * FA_BM;
  if (q0 >= q_len) return;                                  // uniform per CTA, before any set-up
  const int kv_len = p.paged ? p.seq_lens[b] : (p.cu_k[b + 1] - p.cu_k[b]);
  const int k_begin = p.paged ? 0 : p.cu_k[b];
  const int off = kv_len - q_len;                           // key position of query 0
  const int kvh = h / (p.Hq / p.Hkv);
  // keys this tile can see
  int hi = p.causal ? min(kv_len, off + q0 + FA_BM) : kv_len;
  int lo = 0;
  if (p.window > 0) lo = max(0, off + q0 - p.window + 1);
  const int t_begin = lo / FA_BN;
  const int t_end = (hi + FA_BN - 1) / FA_BN;
  const int n_tiles = max(t_end - t_begin, 0);

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t q_s = smem_base;
  const uint32_t kv_s = q_s + Cfg::kTileBytes;
  const uint32_t p_s = kv_s + FA_KV_SLOTS * Cfg::kTileBytes;
  uint8_t* p_ptr = smem_al + Cfg::kTileBytes + FA_KV_SLOTS * Cfg::kTileBytes;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&q_full), 1);
    for (int i = 0; i < FA_KV_SLOTS; ++i) {
      mbar_init(smem_u32(&kv_full[i]), 1);
      mbar_init(smem_u32(&kv_empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&s_full[i]), 1);
      mbar_init(smem_u32(&s_empty[i]), 8);
      mbar_init(smem_u32(&p_full[i]), 8);
      mbar_init(smem_u32(&p_empty[i]), 1);
    }
    for (int i = 0; i < 4; ++i) mbar_init(smem_u32(&xch_bar[i]), 64);
    mbar_init(smem_u32(&o_done), 1);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_smem), FA_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;
  const uint32_t tmem_o = tmem_base + 2 * FA_BN;
  volatile int* abortp = &abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one_sync()) {
      bool ok = true;
      mbar_expect_tx(smem_u32(&q_full), Cfg::kTileBytes);
#pragma unroll
      for (int c = 0; c < DCH; ++c)
        tma_load_2d(q_s + c * CHUNK_BYTES, &p.q_map, smem_u32(&q_full), h * D + c * 64, q_begin + q0);
      uint32_t it = 0;
      // tiles are loaded in the order the MMA warp consumes them: K0, then (K_{j+1}, V_j) for every j
      auto load_tile = [&](int j, int which) -> bool {   // which 0: K tile, 1: V tile
        const int k0 = (t_begin + j) * FA_BN;
        const int slot = it % FA_KV_SLOTS;
        if (!mbar_wait_backoff(smem_u32(&kv_empty[slot]), ((it / FA_KV_SLOTS) & 1u) ^ 1u, abortp, p.status,
                               ST_TIMEOUT_SMEM_EMPTY))
          return false;
        const uint32_t fb = smem_u32(&kv_full[slot]);
        const uint32_t dst = kv_s + slot * Cfg::kTileBytes;
        const CUtensorMap* map = which == 0 ? &p.k_map : &p.v_map;
        mbar_expect_tx(fb, Cfg::kTileBytes);
        if (!p.paged) {
#pragma unroll
          for (int c = 0; c < DCH; ++c) tma_load_2d(dst + c * CHUNK_BYTES, map, fb, kvh * D + c * 64, k_begin + k0);
        } else {
          const int* bt = p.block_tables + (long long)b * p.max_blocks;
          const int n_blk = (kv_len + 15) >> 4;
#pragma unroll 1
          for (int i = 0; i < FA_BN / 16; ++i) {
            const int bi = (k0 >> 4) + i;
            int blk = p.num_blocks;                         // out of range: the copy fills zeros
            if (bi < n_blk) {
              blk = bt[bi];
              if (blk < 0 || blk >= p.num_blocks) { set_status(p.status, ST_BAD_INDEX); blk = p.num_blocks; }
            }
            const int y = (blk * p.Hkv + kvh) * 16;
#pragma unroll
            for (int c = 0; c < DCH; ++c) tma_load_2d(dst + c * CHUNK_BYTES + i * 2048, map, fb, c * 64, y);
          }
        }
        ++it;
        return true;
      };
      if (n_tiles > 0) ok = load_tile(0, 0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) { ok = load_tile(j + 1, 0); if (!ok) break; }
        ok = load_tile(j, 1);
      }
      if (!ok) {   // drain: no bulk copy may land after the CTA has gone
        const uint32_t first = it > (uint32_t)FA_KV_SLOTS ? it - FA_KV_SLOTS : 0;
        for (uint32_t j = first; j < it; ++j) {
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(smem_u32(&kv_full[j % FA_KV_SLOTS]), (j / FA_KV_SLOTS) & 1u))
            if (globaltimer_ns() - t0 > 50000000ull) break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one_sync()) {
      constexpr uint32_t idesc_s = make_idesc_bf16(FA_BM, FA_BN, 0, 0);   // Q, K both K-major
      constexpr uint32_t idesc_o = make_idesc_bf16(FA_BM, D, 0, 1);       // P K-major, V MN-major
      bool ok = mbar_wait_backoff(smem_u32(&q_full), 0, abortp, p.status, ST_TIMEOUT_SMEM_FULL);
      uint32_t it = 0;   // tiles consumed so far, in the producer's order
      auto issue_s = [&](int j) -> bool {
        const int slot = it % FA_KV_SLOTS;
        if (!mbar_wait_backoff(smem_u32(&kv_full[slot]), (it / FA_KV_SLOTS) & 1u, abortp, p.status, ST_TIMEOUT_SMEM_FULL))
          return false;
        if (!mbar_wait_backoff(smem_u32(&s_empty[j & 1]), ((j >> 1) & 1u) ^ 1u, abortp, p.status, ST_TIMEOUT_TMEM_EMPTY))
          return false;
        tc_fence_after();
        const uint32_t ks = kv_s + slot * Cfg::kTileBytes;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint64_t adesc = make_smem_desc_sw128(q_s + (k >> 2) * CHUNK_BYTES + (k & 3) * 32, 16, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(ks + (k >> 2) * CHUNK_BYTES + (k & 3) * 32, 16, 1024);
          umma_bf16(tmem_base + (j & 1) * FA_BN, adesc, bdesc, idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(&kv_empty[slot]));
        umma_commit(smem_u32(&s_full[j & 1]));
        ++it;
        return true;
      };
      if (ok && n_tiles > 0) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) { ok = issue_s(j + 1); if (!ok) break; }
        const int slot = it % FA_KV_SLOTS;
        ok = mbar_wait_backoff(smem_u32(&p_full[j & 1]), (j >> 1) & 1u, abortp, p.status, ST_TIMEOUT_TMEM_FULL);
        if (!ok) break;
        ok = mbar_wait_backoff(smem_u32(&kv_full[slot]), (it / FA_KV_SLOTS) & 1u, abortp, p.status, ST_TIMEOUT_SMEM_FULL);
        if (!ok) break;
        tc_fence_after();
        const uint32_t vs = kv_s + slot * Cfg::kTileBytes;
        const uint32_t ps = p_s + (j & 1) * Cfg::kPBytes;
#pragma unroll
        for (int k = 0; k < FA_BN / 16; ++k) {
          const uint64_t adesc = make_smem_desc_sw128(ps + (k >> 2) * CHUNK_BYTES + (k & 3) * 32, 16, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(vs + k * 2048, CHUNK_BYTES, 1024);
          umma_bf16(tmem_o, adesc, bdesc, idesc_o, (j > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(smem_u32(&kv_empty[slot]));
        umma_commit(smem_u32(&p_empty[j & 1]));
        umma_commit(smem_u32(&o_done));
        ++it;
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    // Two warpgroups (warps 2-5 and 6-9) share the 128 rows: `half` owns 64 of the 128 score columns
    // of a row, half of the O columns and one 64-column chunk of P. The two threads of a row swap
    // their partial row maximum (and, at the end, their partial row sum) through shared memory.
    constexpr int HC = FA_BN / 2;                // score columns per thread
    const int qd = warp & 3;                     // TMEM lane quarter of this warp
    const int half = (warp - 2) >> 2;
    const int r = qd * 32 + lane;                // query row inside the tile
    const uint32_t lane_addr = (uint32_t)(qd * 32) << 16;
    const int qpos = off + q0 + r;               // key position of this query
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    uint32_t xph = 0;                            // phase of the pair barrier
    auto swap_with_partner = [&](float mine, float& other) -> bool {
      xch[xph & 1][half][r] = mine;
      mbar_arrive(smem_u32(&xch_bar[qd]));
      bool good = mbar_wait_backoff(smem_u32(&xch_bar[qd]), xph & 1u, abortp, p.status, ST_TIMEOUT_TMEM_FULL);
      other = xch[xph & 1][half ^ 1][r];
      ++xph;
      return __all_sync(0xffffffffu, good);
    };
    for (int j = 0; j < n_tiles; ++j) {
      const int k0 = (t_begin + j) * FA_BN;
      const uint32_t s_addr = tmem_base + (j & 1) * FA_BN + half * HC + lane_addr;
      ok = mbar_wait_backoff(smem_u32(&s_full[j & 1]), (j >> 1) & 1u, abortp, p.status, ST_TIMEOUT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const bool need_mask = (k0 + FA_BN > kv_len) || (p.causal && k0 + FA_BN - 1 > off + q0) ||
                             (p.window > 0 && k0 <= off + q0 + FA_BM - 1 - p.window);
      // this thread's 64 score columns go to registers with one wait; then the S buffer is free again
      uint32_t v[HC];
#pragma unroll
      for (int c = 0; c < HC / 32; ++c)
        tmem_ld_32x32(s_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&v[c * 32]));
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&s_empty[j & 1]));
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < HC; ++i) {
          const int kj = k0 + half * HC + i;
          const bool dead = kj >= kv_len || (p.causal && kj > qpos) || (p.window > 0 && kj <= qpos - p.window);
          if (dead) v[i] = 0xff800000u;   // -inf
        }
      }
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < HC; i += 4) {
        mx[0] = fmaxf(mx[0], __uint_as_float(v[i]));
        mx[1] = fmaxf(mx[1], __uint_as_float(v[i + 1]));
        mx[2] = fmaxf(mx[2], __uint_as_float(v[i + 2]));
        mx[3] = fmaxf(mx[3], __uint_as_float(v[i + 3]));
      }
      const float mine = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      float other;
      ok = swap_with_partner(mine, other);
      if (!ok) break;
      const float m_new = fmaxf(m_used, fmaxf(mine, other) * p.scale_log2);
      const bool need = m_new > m_used + FA_RESCALE_THRESHOLD || (m_used == -INFINITY && m_new != -INFINITY);
      if (__any_sync(0xffffffffu, need)) {   // same rows, same inputs: both warps of a quarter agree
        if (j > 0) {
          // O holds the products of tiles 0..j-1 once the previous P V has completed
          ok = mbar_wait_backoff(smem_u32(&o_done), (uint32_t)((j - 1) & 1), abortp, p.status, ST_TIMEOUT_TMEM_FULL);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
          const float alpha = need ? fast_exp2((m_used == -INFINITY ? m_new : m_used) - m_new) : 1.f;
#pragma unroll 1
          for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
            uint32_t o[32];
            tmem_ld_32x32(tmem_o + lane_addr + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(tmem_o + lane_addr + c * 32, o);
          }
          tmem_st_wait();
          l *= alpha;
        }
        if (need) m_used = m_new;
      }
      const float mref = m_used == -INFINITY ? 0.f : m_used;
      // P = exp2(S * scale - m): a masked score is -inf and gives exactly 0
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < HC; i += 4) {
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float x = fast_exp2(fmaf(__uint_as_float(v[i + t]), p.scale_log2, -mref));
          ls[t] += x;
          v[i + t] = __float_as_uint(x);
        }
      }
      l += (ls[0] + ls[1]) + (ls[2] + ls[3]);
      // bf16 P into shared memory (A operand of P V) once the P V of two tiles ago has read the buffer
      ok = mbar_wait_backoff(smem_u32(&p_empty[j & 1]), ((j >> 1) & 1u) ^ 1u, abortp, p.status, ST_TIMEOUT_SMEM_EMPTY);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      uint8_t* prow = p_ptr + (j & 1) * Cfg::kPBytes + half * CHUNK_BYTES + r * 128;
#pragma unroll
      for (int unit = 0; unit < HC / 8; ++unit) {
        uint4 w;
        w.x = pack_bf16x2(__uint_as_float(v[unit * 8 + 0]), __uint_as_float(v[unit * 8 + 1]));
        w.y = pack_bf16x2(__uint_as_float(v[unit * 8 + 2]), __uint_as_float(v[unit * 8 + 3]));
        w.z = pack_bf16x2(__uint_as_float(v[unit * 8 + 4]), __uint_as_float(v[unit * 8 + 5]));
        w.w = pack_bf16x2(__uint_as_float(v[unit * 8 + 6]), __uint_as_float(v[unit * 8 + 7]));
        *reinterpret_cast<uint4*>(prow + ((unit ^ (r & 7)) << 4)) = w;
      }
      fence_proxy_async_smem();   // P was written with ordinary stores and is read by the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&p_full[j & 1]));
    }
    if (ok && n_tiles > 0) {
      float l_other;
      ok = swap_with_partner(l, l_other);   // both halves used the same m_used, so the sums simply add
      l += l_other;
    }
    if (ok && n_tiles > 0) {
      ok = mbar_wait_backoff(smem_u32(&o_done), (uint32_t)((n_tiles - 1) & 1), abortp, p.status, ST_TIMEOUT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const bool row_ok = q0 + r < q_len;
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = p.out + ((long long)(q_begin + q0 + r) * p.Hq + h) * D;
#pragma unroll 1
      for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {   // each warpgroup stores half the columns
        uint32_t v[32];
        if (n_tiles > 0) {
          tmem_ld_32x32(tmem_o + lane_addr + c * 32, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(v[u * 8 + 0]) * inv, __uint_as_float(v[u * 8 + 1]) * inv);
            w.y = pack_bf16x2(__uint_as_float(v[u * 8 + 2]) * inv, __uint_as_float(v[u * 8 + 3]) * inv);
            w.z = pack_bf16x2(__uint_as_float(v[u * 8 + 4]) * inv, __uint_as_float(v[u * 8 + 5]) * inv);
            w.w = pack_bf16x2(__uint_as_float(v[u * 8 + 6]) * inv, __uint_as_float(v[u * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + u * 8) = w;
          }
        }
      }
      if (row_ok && half == 0 && p.lse != nullptr)
        p.lse[(long long)h * p.Tq + q_begin + q0 + r] =
            l > 0.f ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
      tc_fence_before();
    }
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, FA_TMEM_COLS);
  }
}


// ------------------------------------------------------------------------------------------
// Forward, two query tiles per CTA ("ping-pong"): 256 query rows of one head, handled as tiles a and b
// with one softmax warpgroup each (warps 2-5 and 6-9, a full score row per thread). Both tiles share the
// K/V tiles in shared memory (loaded once for 256 rows), and while one warpgroup is in its softmax the
// tensor core works for the other tile, so neither the TMEM read, the P store nor the polling of the MMA
// thread sits on a critical path. TMEM: S_a, S_b (128 columns each), O_a, O_b (D columns each).
// ------------------------------------------------------------------------------------------
template <int D>
struct Flash2Cfg {
  static constexpr int kTileBytes = FA_BN * D * 2;
  static constexpr int kPBytes = FA_BM * FA_BN * 2;
  static constexpr int kSmemBytes = 1024 + 2 * kTileBytes + FA_KV_SLOTS * kTileBytes + 2 * kPBytes;
};

template <int D>
__global__ void __launch_bounds__(FA_THREADS, 1) flash_fwd2_kernel(const __grid_constant__ FlashFwdParams p) {
  using Cfg = Flash2Cfg<D>;
  constexpr int DCH = D / 64;
  constexpr int CHUNK_BYTES = FA_BN * 128;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t q_full, kv_full[FA_KV_SLOTS], kv_empty[FA_KV_SLOTS];
  __shared__ __align__(8) uint64_t s_full[2], s_empty[2], p_full[2], p_empty[2], o_done[2];
  __shared__ uint32_t tmem_base_smem;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, h = blockIdx.y;
  const int q_tile = gridDim.x - 1 - blockIdx.x;
  const int q_begin = p.cu_q[b];
  const int q_len = p.cu_q[b + 1] - q_begin;
  const int q0 = q_tile * 2 * FA_BM;
  if (q0 >= q_len) return;
  const int kv_len = p.paged ? p.seq_lens[b] : (p.cu_k[b + 1] - p.cu_k[b]);
  const int k_begin = p.paged ? 0 : p.cu_k[b];
  const int off = kv_len - q_len;
  const int kvh = h / (p.Hq / p.Hkv);
  const bool has_b = q0 + FA_BM < q_len;
  // key tiles: both query tiles start at tile a's first visible tile; each stops at its own last one
  const int lo = p.window > 0 ? max(0, off + q0 - p.window + 1) : 0;
  const int t_begin = lo / FA_BN;
  const int hi_a = p.causal ? min(kv_len, off + q0 + FA_BM) : kv_len;
  const int hi_b = p.causal ? min(kv_len, off + q0 + 2 * FA_BM) : kv_len;
  const int n_a = max((hi_a + FA_BN - 1) / FA_BN - t_begin, 0);
  const int n_b = has_b ? max((hi_b + FA_BN - 1) / FA_BN - t_begin, 0) : 0;
  const int n_tiles = max(n_a, n_b);

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t q_s = smem_base;                                   // Q_a then Q_b
  const uint32_t kv_s = q_s + 2 * Cfg::kTileBytes;
  const uint32_t p_off = 2 * Cfg::kTileBytes + FA_KV_SLOTS * Cfg::kTileBytes;   // P_a then P_b
  const uint32_t p_s = smem_base + p_off;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&q_full), 1);
    for (int i = 0; i < FA_KV_SLOTS; ++i) {
      mbar_init(smem_u32(&kv_full[i]), 1);
      mbar_init(smem_u32(&kv_empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&s_full[i]), 1);
      mbar_init(smem_u32(&s_empty[i]), 4);
      mbar_init(smem_u32(&p_full[i]), 4);
      mbar_init(smem_u32(&p_empty[i]), 1);
      mbar_init(smem_u32(&o_done[i]), 1);
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_smem), FA_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;
  volatile int* abortp = &abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one_sync()) {
      bool ok = true;
      mbar_expect_tx(smem_u32(&q_full), (has_b ? 2 : 1) * Cfg::kTileBytes);
      for (int x = 0; x < (has_b ? 2 : 1); ++x)
#pragma unroll
        for (int c = 0; c < DCH; ++c)
          tma_load_2d(q_s + x * Cfg::kTileBytes + c * CHUNK_BYTES, &p.q_map, smem_u32(&q_full), h * D + c * 64,
                      q_begin + q0 + x * FA_BM);
      uint32_t it = 0;
      auto load_tile = [&](int j, int which) -> bool {
        const int k0 = (t_begin + j) * FA_BN;
        const int slot = it % FA_KV_SLOTS;
        if (!mbar_wait_backoff(smem_u32(&kv_empty[slot]), ((it / FA_KV_SLOTS) & 1u) ^ 1u, abortp, p.status, ST_TIMEOUT_SMEM_EMPTY))
          return false;
        const uint32_t fb = smem_u32(&kv_full[slot]);
        const uint32_t dst = kv_s + slot * Cfg::kTileBytes;
        const CUtensorMap* map = which == 0 ? &p.k_map : &p.v_map;
        mbar_expect_tx(fb, Cfg::kTileBytes);
        if (!p.paged) {
#pragma unroll
          for (int c = 0; c < DCH; ++c) tma_load_2d(dst + c * CHUNK_BYTES, map, fb, kvh * D + c * 64, k_begin + k0);
        } else {
          const int* bt = p.block_tables + (long long)b * p.max_blocks;
          const int n_blk = (kv_len + 15) >> 4;
#pragma unroll 1
          for (int i = 0; i < FA_BN / 16; ++i) {
            const int bi = (k0 >> 4) + i;
            int blk = p.num_blocks;
            if (bi < n_blk) {
              blk = bt[bi];
              if (blk < 0 || blk >= p.num_blocks) { set_status(p.status, ST_BAD_INDEX); blk = p.num_blocks; }
            }
            const int y = (blk * p.Hkv + kvh) * 16;
#pragma unroll
            for (int c = 0; c < DCH; ++c) tma_load_2d(dst + c * CHUNK_BYTES + i * 2048, map, fb, c * 64, y);
          }
        }
        ++it;
        return true;
      };
      if (n_tiles > 0) ok = load_tile(0, 0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) { ok = load_tile(j + 1, 0); if (!ok) break; }
        ok = load_tile(j, 1);
      }
      if (!ok) {
        const uint32_t first = it > (uint32_t)FA_KV_SLOTS ? it - FA_KV_SLOTS : 0;
        for (uint32_t j = first; j < it; ++j) {
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(smem_u32(&kv_full[j % FA_KV_SLOTS]), (j / FA_KV_SLOTS) & 1u))
            if (globaltimer_ns() - t0 > 50000000ull) break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one_sync()) {
      constexpr uint32_t idesc_s = make_idesc_bf16(FA_BM, FA_BN, 0, 0);
      constexpr uint32_t idesc_o = make_idesc_bf16(FA_BM, D, 0, 1);
      bool ok = mbar_wait_backoff(smem_u32(&q_full), 0, abortp, p.status, ST_TIMEOUT_SMEM_FULL);
      uint32_t it = 0;                       // K/V tiles consumed, in the producer's order
      const int n_x[2] = {n_a, n_b};
      // S_x(j) = Q_x K_j^T into TMEM columns x*128; the K tile sits in ring slot `slot`
      auto issue_s = [&](int x, int j, int slot) -> bool {
        if (!mbar_wait_backoff(smem_u32(&s_empty[x]), (uint32_t)((j & 1) ^ 1), abortp, p.status, ST_TIMEOUT_TMEM_EMPTY)) return false;
        tc_fence_after();
        const uint32_t ks = kv_s + slot * Cfg::kTileBytes, qs = q_s + x * Cfg::kTileBytes;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint64_t adesc = make_smem_desc_sw128(qs + (k >> 2) * CHUNK_BYTES + (k & 3) * 32, 16, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(ks + (k >> 2) * CHUNK_BYTES + (k & 3) * 32, 16, 1024);
          umma_bf16(tmem_base + x * FA_BN, adesc, bdesc, idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(&s_full[x]));
        return true;
      };
      auto issue_pv = [&](int x, int j, int slot) -> bool {
        if (!mbar_wait_backoff(smem_u32(&p_full[x]), (uint32_t)(j & 1), abortp, p.status, ST_TIMEOUT_TMEM_FULL)) return false;
        tc_fence_after();
        const uint32_t vs = kv_s + slot * Cfg::kTileBytes, ps = p_s + x * Cfg::kPBytes;
#pragma unroll
        for (int k = 0; k < FA_BN / 16; ++k) {
          const uint64_t adesc = make_smem_desc_sw128(ps + (k >> 2) * CHUNK_BYTES + (k & 3) * 32, 16, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(vs + k * 2048, CHUNK_BYTES, 1024);
          umma_bf16(tmem_base + 2 * FA_BN + x * D, adesc, bdesc, idesc_o, (j > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(smem_u32(&p_empty[x]));
        umma_commit(smem_u32(&o_done[x]));
        return true;
      };
      auto wait_kv = [&](int slot, uint32_t idx) -> bool {
        return mbar_wait_backoff(smem_u32(&kv_full[slot]), (idx / FA_KV_SLOTS) & 1u, abortp, p.status, ST_TIMEOUT_SMEM_FULL);
      };
      if (ok && n_tiles > 0) {
        const int slot = it % FA_KV_SLOTS;
        ok = wait_kv(slot, it);
        if (ok && n_x[0] > 0) ok = issue_s(0, 0, slot);
        if (ok && n_x[1] > 0) ok = issue_s(1, 0, slot);
        if (ok) umma_commit(smem_u32(&kv_empty[slot]));
        ++it;
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        int kslot = -1;
        if (j + 1 < n_tiles) {
          kslot = it % FA_KV_SLOTS;
          ok = wait_kv(kslot, it);
          ++it;
          if (ok && j + 1 < n_x[0]) ok = issue_s(0, j + 1, kslot);
          if (!ok) break;
        }
        const int vslot = it % FA_KV_SLOTS;
        ok = wait_kv(vslot, it);
        ++it;
        if (!ok) break;
        if (j < n_x[0]) { ok = issue_pv(0, j, vslot); if (!ok) break; }
        if (kslot >= 0) {
          if (j + 1 < n_x[1]) { ok = issue_s(1, j + 1, kslot); if (!ok) break; }
          umma_commit(smem_u32(&kv_empty[kslot]));     // K_{j+1} is free once both score products have run
        }
        if (j < n_x[1]) { ok = issue_pv(1, j, vslot); if (!ok) break; }
        umma_commit(smem_u32(&kv_empty[vslot]));
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue, one warpgroup per query tile
    const int x = (warp - 2) >> 2;               // 0: tile a, 1: tile b
    const int qd = warp & 3;
    const int r = qd * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(qd * 32) << 16;
    const int q0x = q0 + x * FA_BM;
    const int qpos = off + q0x + r;
    const int n_mine = x == 0 ? n_a : n_b;
    const uint32_t tmem_s = tmem_base + x * FA_BN + lane_addr;
    const uint32_t tmem_o = tmem_base + 2 * FA_BN + x * D + lane_addr;
    uint8_t* prow = smem_al + p_off + x * Cfg::kPBytes + r * 128;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_mine; ++j) {
      const int k0 = (t_begin + j) * FA_BN;
      ok = mbar_wait_backoff(smem_u32(&s_full[x]), (uint32_t)(j & 1), abortp, p.status, ST_TIMEOUT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const bool need_mask = (k0 + FA_BN > kv_len) || (p.causal && k0 + FA_BN - 1 > off + q0x) ||
                             (p.window > 0 && k0 <= off + q0x + FA_BM - 1 - p.window);
      uint32_t v[FA_BN];
#pragma unroll
      for (int c = 0; c < FA_BN / 32; ++c)
        tmem_ld_32x32(tmem_s + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&v[c * 32]));
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&s_empty[x]));       // the next score product may overwrite S now
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < FA_BN; ++i) {
          const int kj = k0 + i;
          const bool dead = kj >= kv_len || (p.causal && kj > qpos) || (p.window > 0 && kj <= qpos - p.window);
          if (dead) v[i] = 0xff800000u;
        }
      }
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < FA_BN; i += 4) {
        mx[0] = fmaxf(mx[0], __uint_as_float(v[i]));
        mx[1] = fmaxf(mx[1], __uint_as_float(v[i + 1]));
        mx[2] = fmaxf(mx[2], __uint_as_float(v[i + 2]));
        mx[3] = fmaxf(mx[3], __uint_as_float(v[i + 3]));
      }
      const float m_new = fmaxf(m_used, fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2);
      const bool need = m_new > m_used + FA_RESCALE_THRESHOLD || (m_used == -INFINITY && m_new != -INFINITY);
      if (__any_sync(0xffffffffu, need)) {
        if (j > 0) {
          ok = mbar_wait_backoff(smem_u32(&o_done[x]), (uint32_t)((j - 1) & 1), abortp, p.status, ST_TIMEOUT_TMEM_FULL);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
          const float alpha = need ? fast_exp2((m_used == -INFINITY ? m_new : m_used) - m_new) : 1.f;
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(tmem_o + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(tmem_o + c * 32, o);
          }
          tmem_st_wait();
          l *= alpha;
        }
        if (need) m_used = m_new;
      }
      const float mref = m_used == -INFINITY ? 0.f : m_used;
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < FA_BN; i += 4) {
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float e = fast_exp2(fmaf(__uint_as_float(v[i + t]), p.scale_log2, -mref));
          ls[t] += e;
          v[i + t] = __float_as_uint(e);
        }
      }
      l += (ls[0] + ls[1]) + (ls[2] + ls[3]);
      // P buffer is free once the previous P V of this tile has read it
      ok = mbar_wait_backoff(smem_u32(&p_empty[x]), (uint32_t)((j & 1) ^ 1), abortp, p.status, ST_TIMEOUT_SMEM_EMPTY);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
#pragma unroll
      for (int unit = 0; unit < FA_BN / 8; ++unit) {
        uint4 w;
        w.x = pack_bf16x2(__uint_as_float(v[unit * 8 + 0]), __uint_as_float(v[unit * 8 + 1]));
        w.y = pack_bf16x2(__uint_as_float(v[unit * 8 + 2]), __uint_as_float(v[unit * 8 + 3]));
        w.z = pack_bf16x2(__uint_as_float(v[unit * 8 + 4]), __uint_as_float(v[unit * 8 + 5]));
        w.w = pack_bf16x2(__uint_as_float(v[unit * 8 + 6]), __uint_as_float(v[unit * 8 + 7]));
        *reinterpret_cast<uint4*>(prow + (unit >> 3) * CHUNK_BYTES + (((unit & 7) ^ (r & 7)) << 4)) = w;
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&p_full[x]));
    }
    if (ok && n_mine > 0) {
      ok = mbar_wait_backoff(smem_u32(&o_done[x]), (uint32_t)((n_mine - 1) & 1), abortp, p.status, ST_TIMEOUT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok && (x == 0 || has_b)) {
      tc_fence_after();
      const bool row_ok = q0x + r < q_len;
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = p.out + ((long long)(q_begin + q0x + r) * p.Hq + h) * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        if (n_mine > 0) {
          tmem_ld_32x32(tmem_o + c * 32, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(o[u * 8 + 0]) * inv, __uint_as_float(o[u * 8 + 1]) * inv);
            w.y = pack_bf16x2(__uint_as_float(o[u * 8 + 2]) * inv, __uint_as_float(o[u * 8 + 3]) * inv);
            w.z = pack_bf16x2(__uint_as_float(o[u * 8 + 4]) * inv, __uint_as_float(o[u * 8 + 5]) * inv);
            w.w = pack_bf16x2(__uint_as_float(o[u * 8 + 6]) * inv, __uint_as_float(o[u * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + u * 8) = w;
          }
        }
      }
      if (row_ok && p.lse != nullptr)
        p.lse[(long long)h * p.Tq + q_begin + q0x + r] = l > 0.f ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
      tc_fence_before();
    }
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, FA_TMEM_COLS);
  }
}


// ==========================================================================================
// Backward. Three kernels, no atomics, deterministic:
//   prep : delta[h,t] = sum_d dO*O and lse in log2 units
//   dkdv : one CTA per (128-key tile, kv head); loops over the query heads of the group and their
//          64-query tiles. S^T = K Q^T and dP^T = V dO^T land in TMEM (keys on the 128 lanes, so a
//          thread owns a key row), P^T and dS^T go to shared memory as K-major A operands of
//          dV += P^T dO and dK += dS^T Q, which accumulate in TMEM over the whole loop.
//   dq   : one CTA per (128-query tile, head); loops over 64-key tiles. S = Q K^T, dP = dO V^T in
//          TMEM, dS to shared memory, dQ += dS K accumulates in TMEM.
// The same Q / dO / K / V shared-memory tile serves as a K-major operand of the score products and
// as an MN-major operand of the gradient products: only the descriptor differs.
// ==========================================================================================
struct FlashBwdParams {
  CUtensorMap q64, do64, k128, v128;     // dkdv kernel boxes
  CUtensorMap q128, do128, k64, v64;     // dq kernel boxes
  const float* lse2;                     // [Hq, Tq]
  const float* delta;                    // [Hq, Tq]
  __nv_bfloat16 *dq, *dk, *dv;           // [Tq,Hq,D], [Tk,Hkv,D], [Tk,Hkv,D]
  const int* cu_q;
  const int* cu_k;
  int Hq, Hkv, Tq, Tk;
  int causal, window;
  float scale_log2, scale;
  int* status;
  // dK/dV with one CTA per (key tile, QUERY head) instead of per (key tile, key/value head): the CTAs of a group write
  // fp32 partials [2 (dV, dK)][G][Tk][Hkv][D] here and flash_bwd_reduce_kernel sums them in a fixed order. With few
  // long sequences the per-kv-head form leaves most SMs idle behind its longest CTA (G x the query tiles of the
  // first key tile); null = off.
  float* dkv_part;
};

__global__ void flash_bwd_prep_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ out,
                                      const float* __restrict__ lse, float* __restrict__ delta,
                                      float* __restrict__ lse2, int Tq, int Hq, int D) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= Tq * Hq) return;
  const int t = warp / Hq, h = warp % Hq;
  const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(dout + ((long long)t * Hq + h) * D);
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(out + ((long long)t * Hq + h) * D);
  float acc = 0.f;
  for (int i = lane; i < D / 2; i += 32) {
    const float2 x = __bfloat1622float2(a[i]), y = __bfloat1622float2(b[i]);
    acc += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) {
    delta[(long long)h * Tq + t] = acc;
    lse2[(long long)h * Tq + t] = lse[(long long)h * Tq + t] * 1.4426950408889634f;
  }
}

template <int D>
struct FlashBwdCfg {
  static constexpr int kQdoStages = D == 128 ? 2 : 4;       // dkdv: (Q, dO) 64-row tiles in flight
  static constexpr int kKvStages = 3;                       // dq: (K, V) 64-row tiles in flight
  static constexpr int kBig = 128 * D * 2;                  // a 128-row tile
  static constexpr int kSmall = 64 * D * 2;                 // a 64-row tile
  static constexpr int kPd = 128 * 64 * 2;                  // P^T / dS^T / dS tile
  static constexpr int kSmemDkdv = 1024 + 2 * kBig + kQdoStages * 2 * kSmall + 4 * kPd;
  static constexpr int kSmemDq = 1024 + 2 * kBig + kKvStages * 2 * kSmall + 2 * kPd;
};

// 64 packed bf16 values of one row into a 128-byte swizzled row of a K-major tile
__device__ __forceinline__ void store_row64_sw128(uint8_t* row_ptr, int r, const float (&x)[64]) {
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    uint4 w;
    w.x = pack_bf16x2(x[u * 8 + 0], x[u * 8 + 1]);
    w.y = pack_bf16x2(x[u * 8 + 2], x[u * 8 + 3]);
    w.z = pack_bf16x2(x[u * 8 + 4], x[u * 8 + 5]);
    w.w = pack_bf16x2(x[u * 8 + 6], x[u * 8 + 7]);
    *reinterpret_cast<uint4*>(row_ptr + ((u ^ (r & 7)) << 4)) = w;
  }
}

// 32 values (columns half*32 .. half*32+31) of one row into its 128-byte swizzled row
__device__ __forceinline__ void store_row32_sw128(uint8_t* row_ptr, int r, int half, const float (&x)[32]) {
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    uint4 w;
    w.x = pack_bf16x2(x[u * 8 + 0], x[u * 8 + 1]);
    w.y = pack_bf16x2(x[u * 8 + 2], x[u * 8 + 3]);
    w.z = pack_bf16x2(x[u * 8 + 4], x[u * 8 + 5]);
    w.w = pack_bf16x2(x[u * 8 + 6], x[u * 8 + 7]);
    *reinterpret_cast<uint4*>(row_ptr + (((half * 4 + u) ^ (r & 7)) << 4)) = w;
  }
}

// The backward kernels run two softmax warpgroups (warps 2-5 and 6-9): both see the same 128 TMEM
// lanes and split the 64 columns of a tile, which puts two such warps on every scheduler.
constexpr int FA_BWD_THREADS = 320;

template <int D>
__global__ void __launch_bounds__(FA_BWD_THREADS, 1) flash_bwd_dkdv_kernel(const __grid_constant__ FlashBwdParams p) {
  using Cfg = FlashBwdCfg<D>;
  constexpr int DCH = D / 64;
  constexpr int ST = Cfg::kQdoStages;
  constexpr int CH128 = 128 * 128, CH64 = 64 * 128;   // bytes of one 64-column chunk of a 128- / 64-row tile
  extern __shared__ __align__(128) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t kv_full, qdo_full[ST], qdo_empty[ST];
  __shared__ __align__(8) uint64_t st_full[2], st_empty[2], pds_full[2], pds_empty[2], acc_done, stat_bar;
  __shared__ __align__(16) float stat[2][2][64];
  __shared__ uint32_t tmem_base_smem;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Under a causal mask the first key tiles have the longest loops: hand them out first, across all heads (blocks
  // are scheduled in the order of their linear index)
  const int lin = blockIdx.x + gridDim.x * blockIdx.y;
  const int b = blockIdx.z, hy = lin % gridDim.y;
  const int G = p.Hq / p.Hkv;
  const bool head_split = p.dkv_part != nullptr;
  const int kvh = head_split ? hy / G : hy, g_base = head_split ? hy % G : 0;
  const int k_begin = p.cu_k[b], kv_len = p.cu_k[b + 1] - k_begin;
  const int k0 = (lin / gridDim.y) * 128;
  if (k0 >= kv_len) return;
  const int q_begin = p.cu_q[b], q_len = p.cu_q[b + 1] - q_begin;
  const int off = kv_len - q_len;
  // queries that see at least one key of this tile
  const int kmax = min(k0 + 127, kv_len - 1);
  int qi_lo = 0, qi_hi = q_len;
  if (p.causal) qi_lo = max(0, k0 - off);
  if (p.window > 0) qi_hi = min(q_len, kmax + p.window - off);
  const int i_begin = qi_lo / 64;
  const int n_qt = qi_hi > qi_lo ? (qi_hi + 63) / 64 - i_begin : 0;
  const int n_iter = n_qt * (head_split ? 1 : G);

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t k_s = smem_base, v_s = k_s + Cfg::kBig;
  const uint32_t qdo_s = v_s + Cfg::kBig;                       // stage: Q tile then dO tile
  const uint32_t pds_off = 2 * Cfg::kBig + ST * 2 * Cfg::kSmall;   // buffer: P^T then dS^T
  const uint32_t pds_s = smem_base + pds_off;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&kv_full), 1);
    for (int i = 0; i < ST; ++i) { mbar_init(smem_u32(&qdo_full[i]), 1); mbar_init(smem_u32(&qdo_empty[i]), 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&st_full[i]), 1);
      mbar_init(smem_u32(&st_empty[i]), 8);
      mbar_init(smem_u32(&pds_full[i]), 8);
      mbar_init(smem_u32(&pds_empty[i]), 1);
    }
    mbar_init(smem_u32(&acc_done), 1);
    mbar_init(smem_u32(&stat_bar), 256);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_smem), FA_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;
  const uint32_t tm_dv = tmem_base + 256, tm_dk = tmem_base + 256 + D;
  volatile int* abortp = &abort_flag;

  if (warp == 0) {
    if (elect_one_sync()) {
      bool ok = true;
      mbar_expect_tx(smem_u32(&kv_full), 2 * Cfg::kBig);
#pragma unroll
      for (int c = 0; c < DCH; ++c) {
        tma_load_2d(k_s + c * CH128, &p.k128, smem_u32(&kv_full), kvh * D + c * 64, k_begin + k0);
        tma_load_2d(v_s + c * CH128, &p.v128, smem_u32(&kv_full), kvh * D + c * 64, k_begin + k0);
      }
      int it = 0;
      for (; it < n_iter; ++it) {
        const int h = kvh * G + g_base + it / n_qt, i = i_begin + it % n_qt;
        const int stage = it % ST;
        ok = mbar_wait_backoff(smem_u32(&qdo_empty[stage]), ((it / ST) & 1u) ^ 1u, abortp, p.status, ST_TIMEOUT_SMEM_EMPTY);
        if (!ok) break;
        const uint32_t fb = smem_u32(&qdo_full[stage]);
        const uint32_t dst = qdo_s + stage * 2 * Cfg::kSmall;
        mbar_expect_tx(fb, 2 * Cfg::kSmall);
#pragma unroll
        for (int c = 0; c < DCH; ++c) {
          tma_load_2d(dst + c * CH64, &p.q64, fb, h * D + c * 64, q_begin + i * 64);
          tma_load_2d(dst + Cfg::kSmall + c * CH64, &p.do64, fb, h * D + c * 64, q_begin + i * 64);
        }
      }
      if (!ok) {
        for (int j = max(0, it - ST); j < it; ++j) {
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(smem_u32(&qdo_full[j % ST]), (j / ST) & 1u))
            if (globaltimer_ns() - t0 > 50000000ull) break;
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one_sync()) {
      constexpr uint32_t idesc_st = make_idesc_bf16(128, 64, 0, 0);
      constexpr uint32_t idesc_acc = make_idesc_bf16(128, D, 0, 1);
      bool ok = mbar_wait_backoff(smem_u32(&kv_full), 0, abortp, p.status, ST_TIMEOUT_SMEM_FULL);
      auto issue_st = [&](int it) -> bool {
        const int stage = it % ST;
        if (!mbar_wait_backoff(smem_u32(&qdo_full[stage]), (it / ST) & 1u, abortp, p.status, ST_TIMEOUT_SMEM_FULL)) return false;
        if (!mbar_wait_backoff(smem_u32(&st_empty[it & 1]), ((it >> 1) & 1u) ^ 1u, abortp, p.status, ST_TIMEOUT_TMEM_EMPTY)) return false;
        tc_fence_after();
        const uint32_t q_s = qdo_s + stage * 2 * Cfg::kSmall, do_s = q_s + Cfg::kSmall;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint64_t a = make_smem_desc_sw128(k_s + (k >> 2) * CH128 + (k & 3) * 32, 16, 1024);
          const uint64_t bq = make_smem_desc_sw128(q_s + (k >> 2) * CH64 + (k & 3) * 32, 16, 1024);
          umma_bf16(tmem_base + (it & 1) * 64, a, bq, idesc_st, k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint64_t a = make_smem_desc_sw128(v_s + (k >> 2) * CH128 + (k & 3) * 32, 16, 1024);
          const uint64_t bd = make_smem_desc_sw128(do_s + (k >> 2) * CH64 + (k & 3) * 32, 16, 1024);
          umma_bf16(tmem_base + 128 + (it & 1) * 64, a, bd, idesc_st, k > 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(&st_full[it & 1]));
        return true;
      };
      if (ok && n_iter > 0) ok = issue_st(0);
      for (int it = 0; it < n_iter && ok; ++it) {
        if (it + 1 < n_iter) { ok = issue_st(it + 1); if (!ok) break; }
        ok = mbar_wait_backoff(smem_u32(&pds_full[it & 1]), (it >> 1) & 1u, abortp, p.status, ST_TIMEOUT_TMEM_FULL);
        if (!ok) break;
        tc_fence_after();
        const int stage = it % ST;
        const uint32_t q_s = qdo_s + stage * 2 * Cfg::kSmall, do_s = q_s + Cfg::kSmall;
        const uint32_t pt_s = pds_s + (it & 1) * 2 * Cfg::kPd, dst_s = pt_s + Cfg::kPd;
#pragma unroll
        for (int k = 0; k < 4; ++k) {   // 64 queries = 4 k-steps
          const uint64_t a = make_smem_desc_sw128(pt_s + k * 32, 16, 1024);
          const uint64_t bd = make_smem_desc_sw128(do_s + k * 2048, CH64, 1024);
          umma_bf16(tm_dv, a, bd, idesc_acc, (it > 0 || k > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint64_t a = make_smem_desc_sw128(dst_s + k * 32, 16, 1024);
          const uint64_t bq = make_smem_desc_sw128(q_s + k * 2048, CH64, 1024);
          umma_bf16(tm_dk, a, bq, idesc_acc, (it > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(smem_u32(&qdo_empty[stage]));
        umma_commit(smem_u32(&pds_empty[it & 1]));
      }
      if (ok) umma_commit(smem_u32(&acc_done));
    }
  } else {
    const int qd = warp & 3;
    const int r = qd * 32 + lane;                  // key row of the tile
    const int kj = k0 + r;
    const uint32_t lane_addr = (uint32_t)(qd * 32) << 16;
    const int half = (warp - 2) >> 2;              // which 32 of the 64 query columns
    const int tid = threadIdx.x - 64;              // 0..255
    bool ok = true;
    // Row statistics of an iteration's 64 queries (thread t < 64 -> lse2, 64 <= t < 128 -> delta) are fetched one
    // iteration ahead: the loads are issued at the top of iteration it for it + 1 and land in shared memory at its
    // end, so their latency and the 256-thread barrier that publishes them are off the critical path.
    auto load_stat = [&](int it2) -> float {
      const int h2 = kvh * G + g_base + it2 / n_qt, qi = (i_begin + it2 % n_qt) * 64 + (tid & 63);
      const int which = tid >> 6;
      float val = which == 0 ? INFINITY : 0.f;      // lse2 = +inf makes P exactly 0 for rows past the end
      if (qi < q_len) val = (which == 0 ? p.lse2 : p.delta)[(long long)h2 * p.Tq + q_begin + qi];
      return val;
    };
    if (n_iter > 0) {
      if (tid < 128) stat[0][tid >> 6][tid & 63] = load_stat(0);
      mbar_arrive(smem_u32(&stat_bar));
      ok = mbar_wait_backoff(smem_u32(&stat_bar), 0u, abortp, p.status, ST_TIMEOUT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
    }
    for (int it = 0; it < n_iter && ok; ++it) {
      const int qi0 = (i_begin + it % n_qt) * 64;
      const bool have_next = it + 1 < n_iter;
      float stat_next = 0.f;
      if (have_next && tid < 128) stat_next = load_stat(it + 1);
      ok = mbar_wait_backoff(smem_u32(&st_full[it & 1]), (it >> 1) & 1u, abortp, p.status, ST_TIMEOUT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t sv[32], dv[32];
      tmem_ld_32x32(tmem_base + (it & 1) * 64 + half * 32 + lane_addr, sv);
      tmem_ld_32x32(tmem_base + 128 + (it & 1) * 64 + half * 32 + lane_addr, dv);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&st_empty[it & 1]));
      const bool need_mask = (k0 + 127 >= kv_len) || (p.causal && k0 + 127 > off + qi0) ||
                             (p.window > 0 && k0 <= off + qi0 + 63 - p.window);
      const float* l2 = stat[it & 1][0] + half * 32;
      const float* dl = stat[it & 1][1] + half * 32;
      float pr[32], ds[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        float pv = fast_exp2(fmaf(__uint_as_float(sv[c]), p.scale_log2, -l2[c]));
        if (need_mask) {
          const int qpos = off + qi0 + half * 32 + c;
          if (kj >= kv_len || (p.causal && kj > qpos) || (p.window > 0 && kj <= qpos - p.window)) pv = 0.f;
        }
        pr[c] = pv;
        ds[c] = pv * (__uint_as_float(dv[c]) - dl[c]) * p.scale;
      }
      ok = mbar_wait_backoff(smem_u32(&pds_empty[it & 1]), ((it >> 1) & 1u) ^ 1u, abortp, p.status, ST_TIMEOUT_SMEM_EMPTY);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      uint8_t* pt_row = smem_al + pds_off + (it & 1) * 2 * Cfg::kPd + r * 128;
      store_row32_sw128(pt_row, r, half, pr);
      store_row32_sw128(pt_row + Cfg::kPd, r, half, ds);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&pds_full[it & 1]));
      if (have_next) {
        // every thread has read stat[(it + 1) & 1] for the last time in iteration it - 1, before that iteration's barrier
        if (tid < 128) stat[(it + 1) & 1][tid >> 6][tid & 63] = stat_next;
        mbar_arrive(smem_u32(&stat_bar));
        ok = mbar_wait_backoff(smem_u32(&stat_bar), (uint32_t)((it + 1) & 1), abortp, p.status, ST_TIMEOUT_TMEM_FULL);
        ok = __all_sync(0xffffffffu, ok);
      }
    }
    if (ok && n_iter > 0) {
      ok = mbar_wait_backoff(smem_u32(&acc_done), 0, abortp, p.status, ST_TIMEOUT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const bool row_ok = kj < kv_len;
      __nv_bfloat16* dv_row = p.dv + ((long long)(k_begin + kj) * p.Hkv + kvh) * D;
      __nv_bfloat16* dk_row = p.dk + ((long long)(k_begin + kj) * p.Hkv + kvh) * D;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
#pragma unroll 1
        for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {   // each warpgroup stores half the columns
          uint32_t v[32];
          if (n_iter > 0) {
            tmem_ld_32x32((which == 0 ? tm_dv : tm_dk) + lane_addr + c * 32, v);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0u;
          }
          if (row_ok && head_split) {
            float* dst = p.dkv_part + (((long long)(which * G + g_base) * p.Tk + k_begin + kj) * p.Hkv + kvh) * D + c * 32;
#pragma unroll
            for (int u = 0; u < 8; ++u)
              *reinterpret_cast<float4*>(dst + u * 4) = make_float4(__uint_as_float(v[u * 4]), __uint_as_float(v[u * 4 + 1]),
                                                                    __uint_as_float(v[u * 4 + 2]), __uint_as_float(v[u * 4 + 3]));
          } else if (row_ok) {
            __nv_bfloat16* dst = (which == 0 ? dv_row : dk_row) + c * 32;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              uint4 w;
              w.x = pack_bf16x2(__uint_as_float(v[u * 8 + 0]), __uint_as_float(v[u * 8 + 1]));
              w.y = pack_bf16x2(__uint_as_float(v[u * 8 + 2]), __uint_as_float(v[u * 8 + 3]));
              w.z = pack_bf16x2(__uint_as_float(v[u * 8 + 4]), __uint_as_float(v[u * 8 + 5]));
              w.w = pack_bf16x2(__uint_as_float(v[u * 8 + 6]), __uint_as_float(v[u * 8 + 7]));
              *reinterpret_cast<uint4*>(dst + u * 8) = w;
            }
          }
        }
      }
      tc_fence_before();
    }
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, FA_TMEM_COLS);
  }
}

template <int D>
__global__ void __launch_bounds__(FA_BWD_THREADS, 1) flash_bwd_dq_kernel(const __grid_constant__ FlashBwdParams p) {
  using Cfg = FlashBwdCfg<D>;
  constexpr int DCH = D / 64;
  constexpr int ST = Cfg::kKvStages;
  constexpr int CH128 = 128 * 128, CH64 = 64 * 128;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t qdo_full, kv_full[ST], kv_empty[ST];
  __shared__ __align__(8) uint64_t s_full[2], s_empty[2], ds_full[2], ds_empty[2], acc_done;
  __shared__ uint32_t tmem_base_smem;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, h = blockIdx.y;
  const int q_tile = gridDim.x - 1 - blockIdx.x;
  const int q_begin = p.cu_q[b], q_len = p.cu_q[b + 1] - q_begin;
  const int q0 = q_tile * 128;
  if (q0 >= q_len) return;
  const int k_begin = p.cu_k[b], kv_len = p.cu_k[b + 1] - k_begin;
  const int off = kv_len - q_len;
  const int kvh = h / (p.Hq / p.Hkv);
  const int hi = p.causal ? min(kv_len, off + q0 + 128) : kv_len;
  const int lo = p.window > 0 ? max(0, off + q0 - p.window + 1) : 0;
  const int t_begin = lo / 64;
  const int n_iter = max((hi + 63) / 64 - t_begin, 0);

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t q_s = smem_base, do_s = q_s + Cfg::kBig;
  const uint32_t kv_s = do_s + Cfg::kBig;                        // stage: K tile then V tile (64 rows each)
  const uint32_t ds_off = 2 * Cfg::kBig + ST * 2 * Cfg::kSmall;
  const uint32_t ds_s = smem_base + ds_off;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&qdo_full), 1);
    for (int i = 0; i < ST; ++i) { mbar_init(smem_u32(&kv_full[i]), 1); mbar_init(smem_u32(&kv_empty[i]), 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&s_full[i]), 1);
      mbar_init(smem_u32(&s_empty[i]), 8);
      mbar_init(smem_u32(&ds_full[i]), 8);
      mbar_init(smem_u32(&ds_empty[i]), 1);
    }
    mbar_init(smem_u32(&acc_done), 1);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_smem), FA_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;
  const uint32_t tm_dq = tmem_base + 256;
  volatile int* abortp = &abort_flag;

  if (warp == 0) {
    if (elect_one_sync()) {
      bool ok = true;
      mbar_expect_tx(smem_u32(&qdo_full), 2 * Cfg::kBig);
#pragma unroll
      for (int c = 0; c < DCH; ++c) {
        tma_load_2d(q_s + c * CH128, &p.q128, smem_u32(&qdo_full), h * D + c * 64, q_begin + q0);
        tma_load_2d(do_s + c * CH128, &p.do128, smem_u32(&qdo_full), h * D + c * 64, q_begin + q0);
      }
      int it = 0;
      for (; it < n_iter; ++it) {
        const int stage = it % ST;
        ok = mbar_wait_backoff(smem_u32(&kv_empty[stage]), ((it / ST) & 1u) ^ 1u, abortp, p.status, ST_TIMEOUT_SMEM_EMPTY);
        if (!ok) break;
        const uint32_t fb = smem_u32(&kv_full[stage]);
        const uint32_t dst = kv_s + stage * 2 * Cfg::kSmall;
        const int y = k_begin + (t_begin + it) * 64;
        mbar_expect_tx(fb, 2 * Cfg::kSmall);
#pragma unroll
        for (int c = 0; c < DCH; ++c) {
          tma_load_2d(dst + c * CH64, &p.k64, fb, kvh * D + c * 64, y);
          tma_load_2d(dst + Cfg::kSmall + c * CH64, &p.v64, fb, kvh * D + c * 64, y);
        }
      }
      if (!ok) {
        for (int j = max(0, it - ST); j < it; ++j) {
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(smem_u32(&kv_full[j % ST]), (j / ST) & 1u))
            if (globaltimer_ns() - t0 > 50000000ull) break;
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one_sync()) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 64, 0, 0);
      constexpr uint32_t idesc_acc = make_idesc_bf16(128, D, 0, 1);
      bool ok = mbar_wait_backoff(smem_u32(&qdo_full), 0, abortp, p.status, ST_TIMEOUT_SMEM_FULL);
      auto issue_s = [&](int it) -> bool {
        const int stage = it % ST;
        if (!mbar_wait_backoff(smem_u32(&kv_full[stage]), (it / ST) & 1u, abortp, p.status, ST_TIMEOUT_SMEM_FULL)) return false;
        if (!mbar_wait_backoff(smem_u32(&s_empty[it & 1]), ((it >> 1) & 1u) ^ 1u, abortp, p.status, ST_TIMEOUT_TMEM_EMPTY)) return false;
        tc_fence_after();
        const uint32_t k_s = kv_s + stage * 2 * Cfg::kSmall, v_s = k_s + Cfg::kSmall;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint64_t a = make_smem_desc_sw128(q_s + (k >> 2) * CH128 + (k & 3) * 32, 16, 1024);
          const uint64_t bk = make_smem_desc_sw128(k_s + (k >> 2) * CH64 + (k & 3) * 32, 16, 1024);
          umma_bf16(tmem_base + (it & 1) * 64, a, bk, idesc_s, k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint64_t a = make_smem_desc_sw128(do_s + (k >> 2) * CH128 + (k & 3) * 32, 16, 1024);
          const uint64_t bv = make_smem_desc_sw128(v_s + (k >> 2) * CH64 + (k & 3) * 32, 16, 1024);
          umma_bf16(tmem_base + 128 + (it & 1) * 64, a, bv, idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(&s_full[it & 1]));
        return true;
      };
      if (ok && n_iter > 0) ok = issue_s(0);
      for (int it = 0; it < n_iter && ok; ++it) {
        if (it + 1 < n_iter) { ok = issue_s(it + 1); if (!ok) break; }
        ok = mbar_wait_backoff(smem_u32(&ds_full[it & 1]), (it >> 1) & 1u, abortp, p.status, ST_TIMEOUT_TMEM_FULL);
        if (!ok) break;
        tc_fence_after();
        const int stage = it % ST;
        const uint32_t k_s = kv_s + stage * 2 * Cfg::kSmall;
        const uint32_t dsb = ds_s + (it & 1) * Cfg::kPd;
#pragma unroll
        for (int k = 0; k < 4; ++k) {   // 64 keys = 4 k-steps
          const uint64_t a = make_smem_desc_sw128(dsb + k * 32, 16, 1024);
          const uint64_t bk = make_smem_desc_sw128(k_s + k * 2048, CH64, 1024);
          umma_bf16(tm_dq, a, bk, idesc_acc, (it > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(smem_u32(&kv_empty[stage]));
        umma_commit(smem_u32(&ds_empty[it & 1]));
      }
      if (ok) umma_commit(smem_u32(&acc_done));
    }
  } else {
    const int qd = warp & 3;
    const int r = qd * 32 + lane;                  // query row of the tile
    const int half = (warp - 2) >> 2;              // which 32 of the 64 key columns
    const int qi = q0 + r, qpos = off + qi;
    const uint32_t lane_addr = (uint32_t)(qd * 32) << 16;
    float l2 = INFINITY, dl = 0.f;                 // a row past the end gets P = 0 everywhere
    if (qi < q_len) {
      l2 = p.lse2[(long long)h * p.Tq + q_begin + qi];
      dl = p.delta[(long long)h * p.Tq + q_begin + qi];
    }
    bool ok = true;
    for (int it = 0; it < n_iter; ++it) {
      const int k0 = (t_begin + it) * 64;
      ok = mbar_wait_backoff(smem_u32(&s_full[it & 1]), (it >> 1) & 1u, abortp, p.status, ST_TIMEOUT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t sv[32], dv[32];
      tmem_ld_32x32(tmem_base + (it & 1) * 64 + half * 32 + lane_addr, sv);
      tmem_ld_32x32(tmem_base + 128 + (it & 1) * 64 + half * 32 + lane_addr, dv);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&s_empty[it & 1]));
      const bool need_mask = (k0 + 63 >= kv_len) || (p.causal && k0 + 63 > off + q0) ||
                             (p.window > 0 && k0 <= off + q0 + 127 - p.window);
      float ds[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        float pv = fast_exp2(fmaf(__uint_as_float(sv[c]), p.scale_log2, -l2));
        if (need_mask) {
          const int kj = k0 + half * 32 + c;
          if (kj >= kv_len || (p.causal && kj > qpos) || (p.window > 0 && kj <= qpos - p.window)) pv = 0.f;
        }
        ds[c] = pv * (__uint_as_float(dv[c]) - dl) * p.scale;
      }
      ok = mbar_wait_backoff(smem_u32(&ds_empty[it & 1]), ((it >> 1) & 1u) ^ 1u, abortp, p.status, ST_TIMEOUT_SMEM_EMPTY);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      store_row32_sw128(smem_al + ds_off + (it & 1) * Cfg::kPd + r * 128, r, half, ds);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ds_full[it & 1]));
    }
    if (ok && n_iter > 0) {
      ok = mbar_wait_backoff(smem_u32(&acc_done), 0, abortp, p.status, ST_TIMEOUT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const bool row_ok = qi < q_len;
      __nv_bfloat16* dq_row = p.dq + ((long long)(q_begin + qi) * p.Hq + h) * D;
#pragma unroll 1
      for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {   // each warpgroup stores half the columns
        uint32_t v[32];
        if (n_iter > 0) {
          tmem_ld_32x32(tm_dq + lane_addr + c * 32, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(v[u * 8 + 0]), __uint_as_float(v[u * 8 + 1]));
            w.y = pack_bf16x2(__uint_as_float(v[u * 8 + 2]), __uint_as_float(v[u * 8 + 3]));
            w.z = pack_bf16x2(__uint_as_float(v[u * 8 + 4]), __uint_as_float(v[u * 8 + 5]));
            w.w = pack_bf16x2(__uint_as_float(v[u * 8 + 6]), __uint_as_float(v[u * 8 + 7]));
            *reinterpret_cast<uint4*>(dq_row + c * 32 + u * 8) = w;
          }
        }
      }
      tc_fence_before();
    }
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, FA_TMEM_COLS);
  }
}

// dv / dk = sum over the G query heads of a group of their fp32 partials (fixed order), rounded to bf16.
__global__ void flash_bwd_reduce_kernel(const float* __restrict__ part, int G, long long n, __nv_bfloat16* __restrict__ dv,
                                        __nv_bfloat16* __restrict__ dk) {
  const long long nvec = n >> 2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < 2 * nvec; i += (long long)gridDim.x * blockDim.x) {
    const int which = i >= nvec;
    const long long j = which ? i - nvec : i;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int g = 0; g < G; ++g) {
      const float4 v = __ldcs(reinterpret_cast<const float4*>(part + ((long long)which * G + g) * n) + j);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    uint2 o;
    o.x = pack_bf16x2(acc.x, acc.y);
    o.y = pack_bf16x2(acc.z, acc.w);
    reinterpret_cast<uint2*>(which ? dk : dv)[j] = o;
  }
}

template <int D>
static int launch_flash_bwd(const FlashBwdParams& p, dim3 grid_kv, dim3 grid_q, cudaStream_t stream) {
  using Cfg = FlashBwdCfg<D>;
  static bool attr_dev[64] = {};       // the shared-memory opt-in is a per-device function attribute
  int dev_i = 0;
  if (cudaGetDevice(&dev_i) != cudaSuccess || dev_i < 0 || dev_i >= 64) return -10;
  bool& attr = attr_dev[dev_i];
  if (!attr) {
    if (cudaFuncSetAttribute(flash_bwd_dkdv_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemDkdv) !=
        cudaSuccess)
      return -10;
    if (cudaFuncSetAttribute(flash_bwd_dq_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemDq) !=
        cudaSuccess)
      return -10;
    attr = true;
  }
  if (launch_kernel(flash_bwd_dkdv_kernel<D>, grid_kv, dim3(FA_BWD_THREADS), Cfg::kSmemDkdv, stream, p) != cudaSuccess) return -11;
  if (launch_kernel(flash_bwd_dq_kernel<D>, grid_q, dim3(FA_BWD_THREADS), Cfg::kSmemDq, stream, p) != cudaSuccess) return -11;
  if (p.dkv_part != nullptr) {
    const long long n = (long long)p.Tk * p.Hkv * D;
    long long blocks = (2 * (n >> 2) + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    flash_bwd_reduce_kernel<<<(unsigned)blocks, 256, 0, stream>>>(p.dkv_part, p.Hq / p.Hkv, n, p.dv, p.dk);
  }
  return 0;
}

template <int D>
static int launch_flash_fwd(const FlashFwdParams& p, int max_seqlen_q, int B, cudaStream_t stream) {
  static bool attr_dev[64] = {};       // the shared-memory opt-in is a per-device function attribute
  int dev_i = 0;
  if (cudaGetDevice(&dev_i) != cudaSuccess || dev_i < 0 || dev_i >= 64) return -10;
  bool& attr = attr_dev[dev_i];
  if (!attr) {
    if (cudaFuncSetAttribute(flash_fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, FlashCfg<D>::kSmemBytes) != cudaSuccess ||
        cudaFuncSetAttribute(flash_fwd2_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Flash2Cfg<D>::kSmemBytes) != cudaSuccess)
      return -10;
    attr = true;
  }
  static const bool one_tile = getenv("RB_FLASH_ONE_TILE") != nullptr;
  if (max_seqlen_q > FA_BM && !one_tile) {   // two query tiles per CTA share every K/V tile
    dim3 grid((max_seqlen_q + 2 * FA_BM - 1) / (2 * FA_BM), p.Hq, B);
    return launch_kernel(flash_fwd2_kernel<D>, grid, dim3(FA_THREADS), Flash2Cfg<D>::kSmemBytes, stream, p) == cudaSuccess ? 0 : -11;
  }
  dim3 grid((max_seqlen_q + FA_BM - 1) / FA_BM, p.Hq, B);
  return launch_kernel(flash_fwd_kernel<D>, grid, dim3(FA_THREADS), FlashCfg<D>::kSmemBytes, stream, p) == cudaSuccess ? 0 : -11;
}

}  // namespace rb

extern "C" {

// Packed varlen attention forward. Dense mode: k, v are [Tk, Hkv, D] views with row strides
// ldk, ldv (elements) and cu_k gives the key ranges. Paged mode: k, v are the cache
// [num_blocks, Hkv, 16, D] (kv_rows = num_blocks), keys of sequence b are the first seq_lens[b]
// slots of its block table and its queries are the LAST (cu_q[b+1]-cu_q[b]) positions.
int rb_flash_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const int* cu_q,
                 const int* cu_k, const int* seq_lens, const int* block_tables, int B, int Tq, int kv_rows,
                 int Hq, int Hkv, int D, int ldq, int ldk, int ldv, int max_seqlen_q, int max_blocks, int causal,
                 int window, int paged, float scale, int* status, cudaStream_t stream) {
  using namespace rb;
  if (B <= 0 || Tq <= 0 || max_seqlen_q <= 0) return 0;
  if ((D != 64 && D != 128) || Hq % Hkv != 0) return -1;
  FlashFwdParams p;
  if (tma_map_2d_bf16(&p.q_map, q, Tq, (unsigned long long)Hq * D, ldq, FA_BM) != 0) return -20;
  if (!paged) {
    if (tma_map_2d_bf16(&p.k_map, k, kv_rows, (unsigned long long)Hkv * D, ldk, FA_BN) != 0) return -21;
    if (tma_map_2d_bf16(&p.v_map, v, kv_rows, (unsigned long long)Hkv * D, ldv, FA_BN) != 0) return -22;
  } else {
    const unsigned long long rows = (unsigned long long)kv_rows * Hkv * 16;
    if (tma_map_2d_bf16(&p.k_map, k, rows, D, D, 16) != 0) return -21;
    if (tma_map_2d_bf16(&p.v_map, v, rows, D, D, 16) != 0) return -22;
  }
  p.out = (__nv_bfloat16*)out;
  p.lse = lse;
  p.cu_q = cu_q;
  p.cu_k = cu_k;
  p.seq_lens = seq_lens;
  p.block_tables = block_tables;
  p.max_blocks = max_blocks;
  p.num_blocks = paged ? kv_rows : 0;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.Tq = Tq;
  p.causal = causal;
  p.window = window;
  p.paged = paged;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  int rc = D == 64 ? launch_flash_fwd<64>(p, max_seqlen_q, B, stream) : launch_flash_fwd<128>(p, max_seqlen_q, B, stream);
  if (rc != 0) return rc;
  return cudaGetLastError() == cudaSuccess ? 0 : -12;
}

// Backward of rb_flash_fwd in dense mode. out, dout, dq are contiguous [Tq,Hq,D]; dk, dv contiguous
// [Tk,Hkv,D]; workspace holds 2*Hq*Tq floats (delta, lse in log2 units). dkv_part (may be null): 2*(Hq/Hkv)*Tk*Hkv*D
// floats; when given, dK/dV run with one CTA per (key tile, query head) and are reduced over each group afterwards
// (few long sequences: the per-kv-head grid is too coarse to fill the SMs).
int rb_flash_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout, const float* lse,
                 void* dq, void* dk, void* dv, const int* cu_q, const int* cu_k, float* workspace, float* dkv_part, int B, int Tq,
                 int Tk, int Hq, int Hkv, int D, int ldq, int ldk, int ldv, int max_seqlen_q, int max_seqlen_k,
                 int causal, int window, float scale, int* status, cudaStream_t stream) {
  using namespace rb;
  if (B <= 0 || Tq <= 0 || Tk <= 0) return 0;
  if ((D != 64 && D != 128) || Hq % Hkv != 0) return -1;
  FlashBwdParams p;
  const unsigned long long qc = (unsigned long long)Hq * D, kc = (unsigned long long)Hkv * D;
  if (tma_map_2d_bf16(&p.q64, q, Tq, qc, ldq, 64) != 0 || tma_map_2d_bf16(&p.q128, q, Tq, qc, ldq, 128) != 0) return -20;
  if (tma_map_2d_bf16(&p.do64, dout, Tq, qc, qc, 64) != 0 || tma_map_2d_bf16(&p.do128, dout, Tq, qc, qc, 128) != 0) return -21;
  if (tma_map_2d_bf16(&p.k64, k, Tk, kc, ldk, 64) != 0 || tma_map_2d_bf16(&p.k128, k, Tk, kc, ldk, 128) != 0) return -22;
  if (tma_map_2d_bf16(&p.v64, v, Tk, kc, ldv, 64) != 0 || tma_map_2d_bf16(&p.v128, v, Tk, kc, ldv, 128) != 0) return -23;
  float* delta = workspace;
  float* lse2 = workspace + (long long)Hq * Tq;
  p.lse2 = lse2;
  p.delta = delta;
  p.dkv_part = (Hq > Hkv) ? dkv_part : nullptr;
  p.dq = (__nv_bfloat16*)dq;
  p.dk = (__nv_bfloat16*)dk;
  p.dv = (__nv_bfloat16*)dv;
  p.cu_q = cu_q;
  p.cu_k = cu_k;
  p.Hq = Hq; p.Hkv = Hkv; p.Tq = Tq; p.Tk = Tk;
  p.causal = causal; p.window = window;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  const long long warps = (long long)Tq * Hq;
  launch_kernel(flash_bwd_prep_kernel, dim3((unsigned)((warps * 32 + 255) / 256)), dim3(256), 0, stream,
                (const __nv_bfloat16*)dout, (const __nv_bfloat16*)out, lse, delta, lse2, Tq, Hq, D);
  dim3 grid_kv((max_seqlen_k + 127) / 128, p.dkv_part != nullptr ? Hq : Hkv, B), grid_q((max_seqlen_q + 127) / 128, Hq, B);
  int rc = D == 64 ? launch_flash_bwd<64>(p, grid_kv, grid_q, stream) : launch_flash_bwd<128>(p, grid_kv, grid_q, stream);
  if (rc != 0) return rc;
  return cudaGetLastError() == cudaSuccess ? 0 : -12;
}

}  // extern "C"
