// bf16 GEMM for sm_100a on the 5th-generation tensor cores.
//
//   C[M,N] = op(A) * op(B)^T   (fp32 accumulate in TMEM, bf16 or fp32 output)
//
// One persistent CTA per SM. Warp roles:
//   warp 0   : TMA producer (one elected lane) - 128B-swizzled tiles into a multi-stage ring
//   warp 1   : TMEM allocator + tcgen05.mma issuer (one elected lane)
//   warps 2-5: epilogue - tcgen05.ld from TMEM, bias / residual / cast, global or peer stores
// The accumulator is double-buffered in TMEM so the epilogue of tile i overlaps the main
// loop of tile i+1.
//
// Operand majorness: a "K-major" operand is stored [rows, K] with K contiguous (x @ W^T with
// torch Linear weights); an "MN-major" operand is stored [K, rows] with rows contiguous.
// Both are fed by TMA with the 128-byte swizzle and described to the MMA by shared-memory
// descriptors, so forward, dgrad (B MN-major) and wgrad (A and B MN-major) use one kernel.
//
// Peer-partitioned operands: the rows of A (or of B) may be split into `parts` equal slabs,
// each behind its own tensor map. With the maps pointing at other GPUs' symmetric buffers the
// producer warp pulls remote tiles over NVLink tile by tile while the tensor cores work on
// the previous ones: this is the all-gather -> GEMM path (A split: tensor-parallel sequence
// shards; B split: FSDP parameter shards). Only plain tile loads are used for this; no load
// that broadcasts to several CTAs exists in this file.
//
// Reduce epilogues: in EPI_REDUCE_SCATTER / EPI_ALL_REDUCE mode each finished tile is pushed
// with peer stores into the owner GPU's staging slab and published with a release flag; the
// owner's epilogue warps then sum the P partial tiles (their own memory, local reads) and
// write the result (all-reduce: to every peer). This is the GEMM -> reduce-scatter path.
#include "common.cuh"
#include "gemm_sm100.h"

#include <stdlib.h>

#include <mutex>
#include <stdio.h>

namespace rb {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int NUM_ACC = 2;
constexpr int GEMM_THREADS = 192;
constexpr int EPI_WARPS = 4;
// Four norm warps (one tile row per lane) measured 2 % faster per 0.5B decode step than two warps with two rows per
// lane, although 320 threads cap that variant at 168 registers (a few spills in its epilogue): 2.40 vs 2.47 ms,
// 2.45 ms without the fold.
#ifndef RB_NORM_WARPS
#define RB_NORM_WARPS 4
#endif
constexpr int NORM_WARPS = RB_NORM_WARPS;                       // extra warps of a launch with a folded RMSNorm
constexpr int NORM_ROWS = 128 / (NORM_WARPS * 32);  // tile rows per lane of a norm warp
constexpr int GEMM_THREADS_NORM = GEMM_THREADS + NORM_WARPS * 32;
// Launches that carry an all-gather (see GemmParams::gather_*): two extra warps per CTA copy the peers' shards into
// local memory while the tensor cores work. 256 threads keep the full register budget of the plain kernel.
constexpr int GATHER_WARPS = 2;
constexpr int GEMM_THREADS_GATHER = GEMM_THREADS + GATHER_WARPS * 32;
// MN-major 128B-swizzled tiles: 64-element chunks are BK*128 bytes apart (leading offset),
// groups of 8 K-rows are 1024 bytes apart (stride offset).
#ifndef RB_MN_LBO
#define RB_MN_LBO (BK * 128)
#define RB_MN_SBO 1024
#endif

template <int BN>
struct GemmCfg {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // As many stages as fit in 224 KB: small-M GEMMs are bound by TMA round-trip latency divided
  // by the number of loads in flight, so narrow tiles get deep rings (BN=32: 11 stages).
  static constexpr int kStagesFit = (224 * 1024) / kStageBytes;
  static constexpr int kStages = kStagesFit > 12 ? 12 : kStagesFit;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024;
  static constexpr int kTmemCols = (NUM_ACC * BN < 32) ? 32 : NUM_ACC * BN;
};

struct GemmParams {
  CUtensorMap a_map[RB_MAX_PARTS];
  CUtensorMap b_map[RB_MAX_PARTS];
  int M, N, K;            // logical problem (M, N are totals over all parts)
  int a_parts, b_parts;   // row slabs of A / B, one tensor map each
  int a_rows_per_part, b_rows_per_part;
  void* C;                // [M, ldc] bf16 (or fp32 when out_f32)
  long long ldc;
  const __nv_bfloat16* bias;      // [N] or null
  const __nv_bfloat16* residual;  // [M, ldr] or null
  long long ldr;
  int out_f32;
  int epi_mode;           // RB_EPI_*
  // readiness flags for peer-partitioned operands: flag[p] >= epoch before part p is read
  const int* a_ready;
  const int* b_ready;
  int ready_epoch;
  const int* ready_epoch_ptr;   // when set, the epoch to wait for is read from here (graph replay: a device counter)
  // reduce epilogue
  int rank, world;
  void* stage_ptrs[RB_MAX_PARTS];   // peer r's staging base: [world][rows_per_rank][N] bf16
  int* flag_ptrs[RB_MAX_PARTS];     // peer r's flags: [world][tiles_per_rank]
  void* out_ptrs[RB_MAX_PARTS];     // all-reduce: peer r's output [M, ldc]; RS: out_ptrs[rank]
  int reduce_epoch;
  int* status;
  int* epoch_counter;
  int* cta_ticket;
  long long stage_parity_bytes, flag_parity_bytes;
  const int4* tile_table;
  const int* num_tiles_ptr;
  int group_k;            // grouped weight gradient: tiles carry their own K range and output group (see RbGemmArgs::group_mode)
  const unsigned long long* row_dst;
  int swiglu;
  int split_k, kb_per_split;
  int cluster_k;   // split-K slices are the CTAs of one thread-block cluster; partial tiles meet in distributed shared memory
  int red_alias;   // cluster split-K, one work unit per CTA: the partial tile reuses the (drained) TMA ring
  // Folded RMSNorm: C = rstd(row of A) * (A B^T) (+bias), rstd = rsqrt(mean(A[row,:]^2) + eps). Four extra warps
  // read every A tile from the TMA ring as it lands and accumulate the row sums of squares; the caller has
  // multiplied the norm weight into B's columns.
  int norm_fold;
  float norm_eps, norm_inv_k;
  int stages;
  int scaled_epilogue, mirror;
  float alpha, beta;
  int fp8;
  float* sample_ws;
  const float* sample_temperature;
  const unsigned long long* sample_seeds;
  const unsigned long long* sample_step_ptr;
  unsigned long long sample_step_add;
  float* splitk_ws;
  int* splitk_tickets;
  // Fused all-gather of a row-sharded matrix (sharded-parameter training): part r is a contiguous block of
  // gather_part_bytes at gather_src[r] (rank r's shard, peer memory); the two gather warps of every CTA copy an
  // interleaved share of each part to gather_dst + r * gather_part_bytes (local), own part first, and the last CTA
  // to finish a part publishes gather_ready[r] = gather_epoch. When the gathered matrix is this launch's own B
  // operand (b_parts = parts, b_ready = gather_ready), tiles of part r start as soon as part r has landed, and the
  // tile order starts at b_part_rot (the local part). Each remote byte crosses NVLink once.
  const void* gather_src[RB_MAX_PARTS];
  void* gather_dst;
  long long gather_part_bytes;
  int* gather_count;      // [parts] arrival counters, zero between launches
  int* gather_ready;      // [parts]
  int gather_epoch, gather_parts;
  int b_part_rot;
  // The shards may themselves be produced by the peers just before (activations of a tensor-parallel step): a gather
  // warp then waits for gather_src_ready[r] >= the ready epoch before it copies part r. gather_wait_all: the gathered
  // matrix is this launch's A operand as ONE matrix (tiles span the parts), so the producer waits for every part.
  const int* gather_src_ready;
  int gather_wait_all;
};

__device__ __forceinline__ void epi_store_row_chunk(const GemmParams& p, const float* v,
                                                    long long row, int col, int ncols) {
  // v holds 32 fp32 values for (row, col..col+31); ncols valid (multiple of 8).
  if (p.out_f32) {
    float* dst = reinterpret_cast<float*>(p.C) + row * p.ldc + col;
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      if (j < ncols) *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    }
  } else {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + row * p.ldc + col;
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      if (j < ncols) {
        uint4 o;
        o.x = pack_bf16x2(v[j], v[j + 1]);
        o.y = pack_bf16x2(v[j + 2], v[j + 3]);
        o.z = pack_bf16x2(v[j + 4], v[j + 5]);
        o.w = pack_bf16x2(v[j + 6], v[j + 7]);
        *reinterpret_cast<uint4*>(dst + j) = o;
      }
    }
  }
}

// Counter-based random stream of the sampler (identical to rb_sample_logprob: splitmix64 row key,
// murmur3-style 32-bit mixer per column).
__device__ __forceinline__ uint64_t sample_mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
__device__ __forceinline__ uint32_t sample_hash32(uint32_t idx, uint32_t k0, uint32_t k1) {
  uint32_t h = (idx * 0x9E3779B1u) ^ k0;
  h ^= h >> 16; h *= 0x85EBCA6Bu;
  h ^= h >> 13; h *= 0xC2B2AE35u;
  h ^= h >> 16;
  return h + k1;
}

#ifdef RB_GEMM_TIMESTAMPS
// diagnostic build only: per-CTA time stamps of the reduce path, [cta][8]
__device__ unsigned long long g_ts[148 * 8];
#define RB_TS(i) do { if (p.epi_mode != RB_EPI_STORE && threadIdx.x == 64) g_ts[blockIdx.x * 8 + (i)] = globaltimer_ns(); } while (0)
#else
#define RB_TS(i) do { } while (0)
#endif

// NORM = the launch carries the four extra warps of a folded RMSNorm. It is a template parameter because the launch
// bound decides the register budget: 320 threads cap the kernel at 168 registers (with spills in the epilogue),
// 192 threads leave it its 221. Compiling every launch for 320 threads cost the plain GEMMs 4 % (8192^3) and the
// 0.5B decode step 0.1 ms.
template <int BN, bool A_MN, bool B_MN, bool NORM = false, bool GATHER = false>
__global__ void __launch_bounds__(NORM ? GEMM_THREADS_NORM : (GATHER ? GEMM_THREADS_GATHER : GEMM_THREADS), 1)
gemm_bf16_kernel(const __grid_constant__ GemmParams p) {
  static_assert(!(NORM && GATHER), "the extra warps are either norm warps or gather warps");
  using Cfg = GemmCfg<BN>;
  constexpr int MAX_STAGES = Cfg::kStages;
  const int STAGES = p.stages;   // ring depth of this launch (<= MAX_STAGES); short-K launches use a shallow ring
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[MAX_STAGES];
  __shared__ __align__(8) uint64_t empty_bar[MAX_STAGES];
  __shared__ __align__(8) uint64_t tmem_full_bar[NUM_ACC];
  __shared__ __align__(8) uint64_t tmem_empty_bar[NUM_ACC];
  __shared__ __align__(8) uint64_t epi_bar;  // bounded stand-in for a named barrier
  __shared__ uint32_t tmem_base_smem;
  __shared__ int abort_flag;
  __shared__ int splitk_last;
  __shared__ __align__(8) uint64_t red_full_bar;    // cluster split-K: every slice's partial tile is in shared memory
  __shared__ __align__(8) uint64_t red_empty_bar;   // cluster split-K: every peer has finished reading this CTA's partial
  __shared__ __align__(8) uint64_t rs_full_bar[NUM_ACC];   // folded RMSNorm: the row scales of this accumulator are in rs_smem
  __shared__ float rs_smem[NUM_ACC][BM];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  pdl_launch_dependents();  // the next kernel may begin its own prologue now

  const int m_tiles_per_part = (p.a_rows_per_part + BM - 1) / BM;
  const int n_tiles_per_part = (p.b_rows_per_part + BN - 1) / BN;
  const int num_m_tiles = m_tiles_per_part * p.a_parts;
  const int num_n_tiles = n_tiles_per_part * p.b_parts;
  const bool grouped = p.tile_table != nullptr;
  const bool grp = grouped && !p.group_k;   // tiles address rows of A directly (forward and data-gradient forms)
  if (grouped) pdl_wait();  // the tile count itself is produced by the previous kernel
  const int split_k = p.split_k;
  const int num_tiles = (grouped ? *p.num_tiles_ptr : num_m_tiles * num_n_tiles) * split_k;  // work units
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), NORM ? 1 + NORM_WARPS : 1);   // MMA commit (+ the norm warps' reads)
    }
    for (int a = 0; a < NUM_ACC; ++a) {
      mbar_init(smem_u32(&tmem_full_bar[a]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[a]), EPI_WARPS);
      mbar_init(smem_u32(&rs_full_bar[a]), NORM_WARPS);
    }
    mbar_init(smem_u32(&epi_bar), EPI_WARPS * 32);
    if (p.cluster_k) {
      mbar_init(smem_u32(&red_full_bar), split_k * EPI_WARPS);
      mbar_init(smem_u32(&red_empty_bar), split_k * EPI_WARPS);
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_smem), Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (p.cluster_k) cluster_sync_all();   // no peer may signal a barrier that is not initialised yet
  pdl_wait();  // barriers and TMEM are set up; from here on we read what the previous kernel wrote
  RB_TS(0);
  const uint32_t tmem_base = tmem_base_smem;
  volatile int* abortp = &abort_flag;
  // epoch of this reduce call: a host constant, or (graph replay) one past the device counter
  int reduce_epoch = p.reduce_epoch;
  long long stage_off = 0, flag_off = 0;
  if (p.epoch_counter != nullptr) {
    reduce_epoch = ld_relaxed_sys(p.epoch_counter) + 1;
    stage_off = (reduce_epoch & 1) * p.stage_parity_bytes;
    flag_off = (reduce_epoch & 1) * p.flag_parity_bytes;
  }

  // Tile order. In reduce modes, rank r visits the row slab owned by rank r+1 first and its
  // own slab last so that every owner finds its partials early.
  // grouped tiles: m_in = first A row, n_part = first B row, n_in = first output column,
  // m_part carries the number of valid rows
  // kb_lo / kb_hi: the k-blocks of the work unit (a split-K slice, or a group's row range in the grouped weight gradient)
  auto tile_coords = [&](int t, int& m_part, int& m_in, int& n_part, int& n_in, int& kb_lo, int& kb_hi) {
    kb_lo = (t % split_k) * p.kb_per_split;
    kb_hi = split_k > 1 ? min(num_kb, kb_lo + p.kb_per_split) : num_kb;
    t /= split_k;
    if (grouped) {
      const int4 e = p.tile_table[t];
      if (p.group_k) {
        kb_lo = e.x / BK; kb_hi = kb_lo + e.y / BK;
        m_part = e.z; m_in = (e.w >> 16) * BM; n_part = 0; n_in = (e.w & 0xffff) * BN;
        return;
      }
      m_in = e.x; m_part = e.y; n_part = e.z; n_in = e.w;
      return;
    }
    int mt = t % num_m_tiles;
    int nt = t / num_m_tiles;
    if (p.epi_mode != RB_EPI_STORE && p.world > 1) {
      // rotate the slab index
      int slab = mt / m_tiles_per_part;
      int within = mt % m_tiles_per_part;
      slab = (slab + p.rank + 1) % p.a_parts;
      mt = slab * m_tiles_per_part + within;
    }
    m_part = mt / m_tiles_per_part;
    m_in = (mt % m_tiles_per_part) * BM;
    n_part = nt / n_tiles_per_part;
    if (p.b_part_rot) { n_part += p.b_part_rot; if (n_part >= p.b_parts) n_part -= p.b_parts; }   // local shard first
    n_in = (nt % n_tiles_per_part) * BN;
  };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------------------
    if (elect_one_sync()) {
      uint32_t it = 0;
      int ring_s = 0;
      uint32_t ring_ph = 0;
      bool ok = true;
      uint32_t a_seen = 0, b_seen = 0;  // bitmask of parts whose readiness was confirmed
      const int ready_epoch = p.ready_epoch_ptr != nullptr ? *p.ready_epoch_ptr : p.ready_epoch;
      if (GATHER && p.gather_wait_all) {
        // the A operand is the staging matrix as a whole: every part must have landed (decode-sized copies)
        const int gep = p.ready_epoch_ptr != nullptr ? ready_epoch : p.gather_epoch;
        for (int r = 0; r < p.gather_parts && ok; ++r) ok = wait_flag_ge(p.gather_ready + r, gep, p.status);
        if (!ok) *abortp = 1;
        asm volatile("fence.proxy.async.global;" ::: "memory");
      }
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int m_part, m_in, n_part, n_in, kb0, kb1;
        tile_coords(t, m_part, m_in, n_part, n_in, kb0, kb1);
        if (!grouped && p.a_ready != nullptr && !((a_seen >> m_part) & 1u)) {
          ok = wait_flag_ge(p.a_ready + m_part, ready_epoch, p.status);
          if (!ok) { *abortp = 1; break; }
          a_seen |= 1u << m_part;
        }
        if (!grouped && p.b_ready != nullptr && !((b_seen >> n_part) & 1u)) {
          ok = wait_flag_ge(p.b_ready + n_part, ready_epoch, p.status);
          if (!ok) { *abortp = 1; break; }
          // the part may have been written by ordinary stores of this launch's gather warps: order them before
          // the tile loads of the async proxy
          asm volatile("fence.proxy.async.global;" ::: "memory");
          b_seen |= 1u << n_part;
        }
        const CUtensorMap* amap = &p.a_map[grouped ? 0 : m_part];
        const CUtensorMap* bmap = &p.b_map[grouped ? 0 : n_part];
        const int b_row = (grp && !B_MN) ? n_part : n_in;   // first B row (K-major) or column (MN-major) of the tile
        const int b_k0 = (grp && B_MN) ? n_part : 0;        // grouped data gradient: the group's first row of the stacked B
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          // ring slot and phase advance incrementally: the depth is a run-time value, and a division per k-block sat
          // on the single-thread critical path of this role
          const int s = ring_s;
          const uint32_t ph = ring_ph;
          if (++ring_s == STAGES) { ring_s = 0; ring_ph ^= 1u; }
          ok = mbar_wait_bounded(smem_u32(&empty_bar[s]), ph ^ 1u, abortp, p.status,
                                 ST_TIMEOUT_SMEM_EMPTY);
          if (!ok) break;
          const uint32_t fb = smem_u32(&full_bar[s]);
          const uint32_t sa = smem_base + s * Cfg::kStageBytes;
          const uint32_t sb = sa + Cfg::kABytes;
          mbar_expect_tx(fb, Cfg::kStageBytes);
          if (!A_MN) {
            tma_load_2d(sa, amap, fb, kb * BK, m_in);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d(sa + c * (BK * 128), amap, fb, m_in + c * 64, kb * BK);
          }
          if (!B_MN) {
            tma_load_2d(sb, bmap, fb, kb * BK, b_row);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_2d(sb + c * (BK * 128), bmap, fb, b_row + c * 64, b_k0 + kb * BK);
          }
        }
      }
      // Drain: never leave the CTA with bulk copies still landing in its shared memory.
      if (!ok) {
        const uint32_t issued = it;
        const uint32_t first = issued > (uint32_t)STAGES ? issued - STAGES : 0;
        for (uint32_t j = first; j < issued; ++j) {
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(smem_u32(&full_bar[j % STAGES]), (j / STAGES) & 1u)) {
            if (globaltimer_ns() - t0 > 50000000ull) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------------------
    if (elect_one_sync()) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      const uint32_t idesc8 = make_idesc_f8(BM, BN, (p.fp8 >> 1) & 1, (p.fp8 >> 2) & 1);
      uint32_t it = 0;
      int ring_s = 0;
      uint32_t ring_ph = 0;
      uint32_t tile_iter = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_iter) {
        const int acc = tile_iter % NUM_ACC;
        const uint32_t acc_ph = (tile_iter / NUM_ACC) & 1u;
        ok = mbar_wait_bounded(smem_u32(&tmem_empty_bar[acc]), acc_ph ^ 1u, abortp, p.status,
                               ST_TIMEOUT_TMEM_EMPTY);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        int kb0 = (t % split_k) * p.kb_per_split;
        int kb1 = split_k > 1 ? min(num_kb, kb0 + p.kb_per_split) : num_kb;
        if (p.group_k) {
          const int4 e = p.tile_table[t];
          kb0 = e.x / BK; kb1 = kb0 + e.y / BK;
        }
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          // ring slot and phase advance incrementally: the depth is a run-time value, and a division per k-block sat
          // on the single-thread critical path of this role
          const int s = ring_s;
          const uint32_t ph = ring_ph;
          if (++ring_s == STAGES) { ring_s = 0; ring_ph ^= 1u; }
          ok = mbar_wait_bounded(smem_u32(&full_bar[s]), ph, abortp, p.status,
                                 ST_TIMEOUT_SMEM_FULL);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_base + s * Cfg::kStageBytes;
          const uint32_t sb = sa + Cfg::kABytes;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = A_MN ? make_smem_desc_sw128(sa + k * 2048, RB_MN_LBO, RB_MN_SBO)
                                        : make_smem_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc_sw128(sb + k * 2048, RB_MN_LBO, RB_MN_SBO)
                                        : make_smem_desc_sw128(sb + k * 32, 16, 1024);
            if (p.fp8) umma_f8(tmem_d, adesc, bdesc, idesc8, (kb > kb0 || k > 0) ? 1u : 0u);
            else umma_bf16(tmem_d, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(smem_u32(&empty_bar[s]));  // frees the stage when these MMAs retire
        }
        if (ok) umma_commit(smem_u32(&tmem_full_bar[acc]));
      }
    }
  } else if (GATHER && warp >= 2 + EPI_WARPS) {
    // ------------------------------ gather warps (fused all-gather only) ---------------------
    constexpr int GT = GATHER_WARPS * 32;
    const int gt = (warp - 2 - EPI_WARPS) * 32 + lane;
    const long long nvec = p.gather_part_bytes >> 4;
    const long long stride = (long long)gridDim.x * GT;
    const int src_epoch = p.ready_epoch_ptr != nullptr ? *p.ready_epoch_ptr : p.ready_epoch;
    const int gather_epoch = p.ready_epoch_ptr != nullptr ? src_epoch : p.gather_epoch;
    __shared__ int gather_failed;
    if (gt == 0) gather_failed = 0;
    asm volatile("bar.sync 1, %0;" ::"n"(GT) : "memory");
    for (int pp = 0; pp < p.gather_parts; ++pp) {
      int part = p.rank + pp;
      if (part >= p.gather_parts) part -= p.gather_parts;
      if (p.gather_src_ready != nullptr && part != p.rank) {
        // the owner of this part publishes it with a flag: wait (bounded) before the first byte is read
        if (gt == 0 && !wait_flag_ge(p.gather_src_ready + part, src_epoch, p.status)) gather_failed = 1;
        asm volatile("bar.sync 1, %0;" ::"n"(GT) : "memory");
        if (gather_failed) break;
      }
      const uint4* src = reinterpret_cast<const uint4*>(p.gather_src[part]);
      uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<char*>(p.gather_dst) + (long long)part * p.gather_part_bytes);
      constexpr int U = 8;     // eight 16-byte loads in flight per thread: the copy is bound by NVLink latency otherwise
      for (long long i0 = (long long)blockIdx.x * GT + gt; i0 < nvec; i0 += stride * U) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + u * stride;
          if (i < nvec)
            asm volatile("ld.global.relaxed.sys.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w) : "l"(src + i) : "memory");
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + u * stride;
          if (i < nvec) dst[i] = v[u];
        }
      }
      __threadfence();
      asm volatile("fence.proxy.async.global;" ::: "memory");
      asm volatile("bar.sync 1, %0;" ::"n"(GT) : "memory");    // the gather warps of this CTA only
      if (gt == 0) {
        const int old = atomicAdd(p.gather_count + part, 1);
        if (old == (int)gridDim.x - 1) {     // every CTA's share of this part is in place
          p.gather_count[part] = 0;
          __threadfence();
          st_release_sys(p.gather_ready + part, gather_epoch);
        }
      }
    }
  } else if (warp >= 2 + EPI_WARPS) {
    // ------------------------------ norm warps (folded RMSNorm only) -----------------------
    // NORM_ROWS tile rows per lane: as each A tile lands in the ring, add the squares of its 64 values of those
    // rows (a row is 128 contiguous bytes whose 16-byte chunks are permuted by the swizzle, which a sum ignores).
    const int nrow = (warp - 2 - EPI_WARPS) * (NORM_ROWS * 32) + lane;
    uint32_t it = 0, tile_iter = 0;
    int ring_s = 0;
    uint32_t ring_ph = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_iter) {
      const int acc = tile_iter % NUM_ACC;
      const uint32_t acc_ph = (tile_iter / NUM_ACC) & 1u;
      // rs_smem[acc] was read by the epilogue of the tile that last used this accumulator
      ok = mbar_wait_bounded(smem_u32(&tmem_empty_bar[acc]), acc_ph ^ 1u, abortp, p.status, ST_TIMEOUT_TMEM_EMPTY);
      if (!ok) break;
      float ss[NORM_ROWS][4];   // four chains per row: the sums must not serialise
#pragma unroll
      for (int r = 0; r < NORM_ROWS; ++r) ss[r][0] = ss[r][1] = ss[r][2] = ss[r][3] = 0.f;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = ring_s;
        const uint32_t ph = ring_ph;
        if (++ring_s == STAGES) { ring_s = 0; ring_ph ^= 1u; }
        ok = mbar_wait_bounded(smem_u32(&full_bar[s]), ph, abortp, p.status, ST_TIMEOUT_SMEM_FULL);
        if (!ok) break;
        const uint8_t* arow = smem_raw + (smem_base - smem_u32(smem_raw)) + (size_t)s * Cfg::kStageBytes + (size_t)nrow * 128;
        uint4 c[NORM_ROWS][8];
#pragma unroll
        for (int r = 0; r < NORM_ROWS; ++r)
#pragma unroll
          for (int j = 0; j < 8; ++j) c[r][j] = *reinterpret_cast<const uint4*>(arow + r * 32 * 128 + ((j ^ (lane & 7)) << 4));
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&empty_bar[s]));   // the rows are in registers: release the stage first
#pragma unroll
        for (int r = 0; r < NORM_ROWS; ++r)
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float2 f;
            f = unpack_bf16x2(c[r][j].x); ss[r][0] = fmaf(f.x, f.x, ss[r][0]); ss[r][1] = fmaf(f.y, f.y, ss[r][1]);
            f = unpack_bf16x2(c[r][j].y); ss[r][2] = fmaf(f.x, f.x, ss[r][2]); ss[r][3] = fmaf(f.y, f.y, ss[r][3]);
            f = unpack_bf16x2(c[r][j].z); ss[r][0] = fmaf(f.x, f.x, ss[r][0]); ss[r][1] = fmaf(f.y, f.y, ss[r][1]);
            f = unpack_bf16x2(c[r][j].w); ss[r][2] = fmaf(f.x, f.x, ss[r][2]); ss[r][3] = fmaf(f.y, f.y, ss[r][3]);
          }
      }
      if (!ok) break;
#pragma unroll
      for (int r = 0; r < NORM_ROWS; ++r)
        rs_smem[acc][nrow + r * 32] = rsqrtf(((ss[r][0] + ss[r][1]) + (ss[r][2] + ss[r][3])) * p.norm_inv_k + p.norm_eps);
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&rs_full_bar[acc]));
    }
  } else {
    // ------------------------------ epilogue warps ----------------------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    // reduce modes: a [32 rows][BN columns] bf16 slab per epilogue warp behind the TMA ring (row pitch
    // padded by 16 bytes so that the row-per-lane writes spread over the banks)
    constexpr int EPI_ROWB = BN * 2 + 16;
    uint8_t* epi_stage = smem_raw + (smem_base - smem_u32(smem_raw)) + (size_t)STAGES * Cfg::kStageBytes +
                         (size_t)(warp - 2) * 32 * EPI_ROWB;
    uint32_t tile_iter = 0;
    bool ok = true;
    uint32_t epi_phase = 0;
    // Barrier over the 128 epilogue threads whose wait is bounded: if some thread has left
    // the loop after a timeout, the others give up too instead of hanging.
    auto epi_sync = [&]() -> bool {
      mbar_arrive(smem_u32(&epi_bar));
      bool r = mbar_wait_bounded(smem_u32(&epi_bar), epi_phase, abortp, p.status, ST_TIMEOUT_TMEM_FULL);
      epi_phase ^= 1u;
      return r;
    };
    const int rows_per_rank = p.a_rows_per_part;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_iter) {
      int m_part, m_in, n_part, n_in, kb_lo_, kb_hi_;
      tile_coords(t, m_part, m_in, n_part, n_in, kb_lo_, kb_hi_);
      const int acc = tile_iter % NUM_ACC;
      const uint32_t acc_ph = (tile_iter / NUM_ACC) & 1u;
      ok = mbar_wait_bounded(smem_u32(&tmem_full_bar[acc]), acc_ph, abortp, p.status,
                             ST_TIMEOUT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
      RB_TS(1);
      float rscale = 1.f;
      if constexpr (NORM) {
        ok = mbar_wait_bounded(smem_u32(&rs_full_bar[acc]), acc_ph, abortp, p.status, ST_TIMEOUT_SMEM_FULL);
        if (!ok) break;
        rscale = rs_smem[acc][q * 32 + lane];
      }
      const int row_in = m_in + q * 32 + lane;                 // row inside the A slab
      const bool row_ok = grp ? (q * 32 + lane < m_part) : (row_in < p.a_rows_per_part);
      const long long row = grp ? (long long)row_in : (long long)m_part * p.a_rows_per_part + row_in;
      const int n_base = grp ? n_in : n_part * p.b_rows_per_part + n_in;    // global column
      const int n_valid = min(BN, p.b_rows_per_part - n_in);   // columns valid in this tile
      if (p.cluster_k) {
        // ---- cluster split-K: the split_k CTAs of a cluster each hold the fp32 partial tile of one K slice.
        // Every CTA parks its partial in its own shared memory, then reduces and stores one column slice of
        // the tile, reading the peers' partials through distributed shared memory (fixed slice order, so the
        // sum is deterministic). No global workspace, no tickets.
        const int S = split_k;
        const int ks = t % S;   // == rank of this CTA in its cluster (the grid is a multiple of S)
        const int trow = q * 32 + lane;
        // behind the ring, or (one unit per CTA: every load has landed and every MMA has retired once the
        // accumulator is complete) on top of it
        const uint32_t red_off = p.red_alias ? 0u : (uint32_t)STAGES * Cfg::kStageBytes;
        const uint32_t red_u32 = smem_base + red_off;
        float4* red = reinterpret_cast<float4*>(smem_raw + (smem_base - smem_u32(smem_raw)) + red_off);
        if (tile_iter > 0) {   // the peers must have finished reading the previous partial
          ok = mbar_wait_bounded_cluster(smem_u32(&red_empty_bar), (tile_iter - 1) & 1u, abortp, p.status, ST_TIMEOUT_TMEM_EMPTY);
          if (!ok) break;
        }
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + acc * BN + c0 + ((uint32_t)(q * 32) << 16), r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            red[((c0 + j) >> 2) * BM + trow] = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                          __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[acc]));
        fence_acq_rel_cluster();
        __syncwarp();
        if (lane < S) mbar_arrive_cluster(mapa_cluster(smem_u32(&red_full_bar), (uint32_t)lane));
        ok = mbar_wait_bounded_cluster(smem_u32(&red_full_bar), tile_iter & 1u, abortp, p.status, ST_TIMEOUT_TMEM_FULL);
        if (!ok) break;
        const int W = BN / S;   // columns this CTA finishes (a multiple of 8)
#pragma unroll 1
        for (int w0 = 0; w0 < W; w0 += 32) {
          const int wn = min(32, W - w0);
          const int cbase = ks * W + w0;            // first column inside the tile
          const int ncols = min(wn, n_valid - cbase);
          if (ncols <= 0) break;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0.f;
#pragma unroll 1
          for (int s2 = 0; s2 < S; ++s2) {
            const uint32_t peer = mapa_cluster(red_u32, (uint32_t)s2);
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (j < wn) {
                const float4 f = ld_dsmem_f4(peer + (uint32_t)((((cbase + j) >> 2) * BM + trow) * 16));
                v[j] += f.x; v[j + 1] += f.y; v[j + 2] += f.z; v[j + 3] += f.w;
              }
            }
          }
          if (row_ok) {
            const int col = n_base + cbase;
            if (p.bias != nullptr) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (j < ncols) v[j] += __bfloat162float(p.bias[col + j]);
            }
            if (p.residual != nullptr) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (j < ncols) v[j] += __bfloat162float(p.residual[row * p.ldr + col + j]);
            }
            epi_store_row_chunk(p, v, row, col, ncols);
          }
        }
        fence_acq_rel_cluster();
        __syncwarp();
        if (lane < S) mbar_arrive_cluster(mapa_cluster(smem_u32(&red_empty_bar), (uint32_t)lane));
        continue;
      }
      if (split_k > 1) {
        // ---- split-K: fp32 partial tile -> workspace; the last slice to arrive finishes the tile ----
        // Workspace layout per work unit: [BN/4 column quads][BM rows] of float4, so that the 32
        // lanes of a warp (32 consecutive rows) store and load 512 contiguous bytes.
        constexpr int UNIT_F4 = BM * BN / 4;
        const int ks = t % split_k;
        const int trow = q * 32 + lane;
        float4* wsu = reinterpret_cast<float4*>(p.splitk_ws) + (long long)t * UNIT_F4;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + acc * BN + c0 + ((uint32_t)(q * 32) << 16), r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            wsu[((c0 + j) >> 2) * BM + trow] = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                          __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[acc]));
        __threadfence();
        ok = epi_sync();
        if (!ok) break;
        if (warp == 2 && lane == 0) {
          const int tk = atomicAdd(&p.splitk_tickets[t / split_k], 1);
          splitk_last = (tk == split_k - 1) ? 1 : 0;
          if (tk == split_k - 1) p.splitk_tickets[t / split_k] = 0;  // ready for the next launch
        }
        ok = epi_sync();
        if (!ok) break;
        if (splitk_last) {
          __threadfence();
          const float4* base = reinterpret_cast<const float4*>(p.splitk_ws) + (long long)(t - ks) * UNIT_F4;
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 32) {
            const int ncols = min(32, n_valid - c0);
            if (ncols <= 0) break;
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0.f;
#pragma unroll 4
            for (int s2 = 0; s2 < split_k; ++s2) {   // fixed order: the sum does not depend on arrival order
              const float4* src = base + (long long)s2 * UNIT_F4 + (c0 >> 2) * BM + trow;
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                const float4 f = __ldcg(src + (j >> 2) * BM);
                v[j] += f.x; v[j + 1] += f.y; v[j + 2] += f.z; v[j + 3] += f.w;
              }
            }
            if (row_ok) {
              const int col = n_base + c0;
              if (p.bias != nullptr) {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (j < ncols) v[j] += __bfloat162float(p.bias[col + j]);
              }
              if (p.residual != nullptr) {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (j < ncols) v[j] += __bfloat162float(p.residual[row * p.ldr + col + j]);
              }
              epi_store_row_chunk(p, v, row, col, ncols);
            }
          }
        }
        ok = epi_sync();   // splitk_last is reused by the next unit
        if (!ok) break;
        continue;
      }
      if (p.sample_ws != nullptr) {
        // ---- fused sampling: reduce this tile's logits per row, store one record per (row, n tile) ----
        float temp = 1.f;
        uint32_t k0 = 0, k1 = 0;
        if (row_ok) {
          temp = p.sample_temperature[row];
          const unsigned long long step = p.sample_step_add + (p.sample_step_ptr != nullptr ? *p.sample_step_ptr : 0ull);
          const uint64_t key = sample_mix64(sample_mix64(p.sample_seeds[row]) ^ (step * 0x9E3779B97F4A7C15ull));
          k0 = (uint32_t)key; k1 = (uint32_t)(key >> 32);
        }
        const bool greedy = temp <= 0.f;
        const float inv_t = greedy ? 1.f : 1.f / temp;
        float m = -INFINITY, ssum = 0.f, best = -INFINITY, best_logit = 0.f;
        int best_i = 0x7fffffff;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + acc * BN + c0 + ((uint32_t)(q * 32) << 16), r);
          tmem_ld_wait();
          const int ncols = min(32, n_valid - c0);
          if (ncols <= 0) break;
          float m4 = -INFINITY;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < ncols) m4 = fmaxf(m4, __uint_as_float(r[j]));
          if (m4 > m) { ssum *= __expf(m - m4); m = m4; }
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (j < ncols) {
              const float x = __uint_as_float(r[j]);
              ssum += __expf(x - m);
              float score = x * inv_t;
              if (!greedy) {
                const uint32_t h = sample_hash32((uint32_t)(n_base + c0 + j), k0, k1);
                const float u = ((float)(h >> 8) + 0.5f) * (1.0f / 16777216.0f);
                score -= 0.6931471805599453f * __log2f(-0.6931471805599453f * __log2f(u));
              }
              if (score > best) { best = score; best_i = n_base + c0 + j; best_logit = x; }
            }
          }
        }
        if (row_ok) {
          float4* rec = reinterpret_cast<float4*>(p.sample_ws) + ((long long)row * num_n_tiles + n_in / BN) * 2;
          rec[0] = make_float4(m, ssum, best, best_logit);
          rec[1] = make_float4(__int_as_float(best_i), 0.f, 0.f, 0.f);
        }
      } else if (p.swiglu) {
        if constexpr (BN >= 64) {
          // gate columns [0, BN/2), up columns [BN/2, BN) of the same output channels
          const int out_col0 = (n_base / BN) * (BN / 2);
#pragma unroll 1
          for (int c0 = 0; c0 < BN / 2; c0 += 32) {
            uint32_t g[32], u[32];
            tmem_ld_32x32(tmem_base + acc * BN + c0 + ((uint32_t)(q * 32) << 16), g);
            tmem_ld_32x32(tmem_base + acc * BN + BN / 2 + c0 + ((uint32_t)(q * 32) << 16), u);
            tmem_ld_wait();
            if (row_ok) {
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + row * p.ldc + out_col0 + c0;
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint32_t o[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  // same rounding points as the unfused path: bf16(gate), bf16(silu), bf16(up), bf16(product)
                  const float g0 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(g[j + 2 * e]) * rscale));
                  const float g1 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(g[j + 2 * e + 1]) * rscale));
                  const float u0 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(u[j + 2 * e]) * rscale));
                  const float u1 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(u[j + 2 * e + 1]) * rscale));
                  const float s0 = __bfloat162float(__float2bfloat16_rn(g0 / (1.f + __expf(-g0))));
                  const float s1 = __bfloat162float(__float2bfloat16_rn(g1 / (1.f + __expf(-g1))));
                  o[e] = pack_bf16x2(s0 * u0, s1 * u1);
                }
                *reinterpret_cast<uint4*>(dst + j) = make_uint4(o[0], o[1], o[2], o[3]);
              }
            }
          }
        }
      } else
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + acc * BN + c0 + ((uint32_t)(q * 32) << 16), r);
        tmem_ld_wait();
        const int ncols = min(32, n_valid - c0);
        if (row_ok && ncols > 0) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * rscale;
          const int col = n_base + c0;
          if (p.scaled_epilogue) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= p.alpha;
          }
          if (p.epi_mode == RB_EPI_STORE) {
            if (p.bias != nullptr) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                if (j < ncols) {
                  uint4 b = *reinterpret_cast<const uint4*>(p.bias + col + j);
                  float2 f;
                  f = unpack_bf16x2(b.x); v[j] += f.x; v[j + 1] += f.y;
                  f = unpack_bf16x2(b.y); v[j + 2] += f.x; v[j + 3] += f.y;
                  f = unpack_bf16x2(b.z); v[j + 4] += f.x; v[j + 5] += f.y;
                  f = unpack_bf16x2(b.w); v[j + 6] += f.x; v[j + 7] += f.y;
                }
              }
            }
            if (p.residual != nullptr) {
              const __nv_bfloat16* rp = p.residual + row * p.ldr + col;
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                if (j < ncols) {
                  uint4 b = *reinterpret_cast<const uint4*>(rp + j);
                  const float rs = p.scaled_epilogue ? p.beta : 1.f;
                  float2 f;
                  f = unpack_bf16x2(b.x); v[j] = fmaf(rs, f.x, v[j]); v[j + 1] = fmaf(rs, f.y, v[j + 1]);
                  f = unpack_bf16x2(b.y); v[j + 2] = fmaf(rs, f.x, v[j + 2]); v[j + 3] = fmaf(rs, f.y, v[j + 3]);
                  f = unpack_bf16x2(b.z); v[j + 4] = fmaf(rs, f.x, v[j + 4]); v[j + 5] = fmaf(rs, f.y, v[j + 5]);
                  f = unpack_bf16x2(b.w); v[j + 6] = fmaf(rs, f.x, v[j + 6]); v[j + 7] = fmaf(rs, f.y, v[j + 7]);
                }
              }
            }
            if (p.row_dst != nullptr) {
              // fused combine: this row's home is an arbitrary (possibly remote) address
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.row_dst[row]) + col;
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                if (j < ncols) {
                  uint4 o;
                  o.x = pack_bf16x2(v[j], v[j + 1]);
                  o.y = pack_bf16x2(v[j + 2], v[j + 3]);
                  o.z = pack_bf16x2(v[j + 4], v[j + 5]);
                  o.w = pack_bf16x2(v[j + 6], v[j + 7]);
                  *reinterpret_cast<uint4*>(dst + j) = o;
                }
              }
            } else {
              epi_store_row_chunk(p, v, row, col, ncols);
              if (p.mirror) {
                // transposed copy of the part below the diagonal: for a fixed j the lanes of a warp
                // (consecutive rows) write consecutive addresses
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  if (j < ncols && col + j < row) {
                    if (p.out_f32) reinterpret_cast<float*>(p.C)[(long long)(col + j) * p.ldc + row] = v[j];
                    else reinterpret_cast<__nv_bfloat16*>(p.C)[(long long)(col + j) * p.ldc + row] = __float2bfloat16_rn(v[j]);
                  }
                }
              }
            }
          } else {
            // reduce modes: park the bf16 partial in this warp's shared-memory slab; the rows are sent to
            // the peers below with lane-contiguous stores (a thread-per-row store would cross NVLink as
            // 16-byte packets)
            uint8_t* srow = epi_stage + (size_t)lane * EPI_ROWB + c0 * 2;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 o;
              o.x = pack_bf16x2(v[j], v[j + 1]);
              o.y = pack_bf16x2(v[j + 2], v[j + 3]);
              o.z = pack_bf16x2(v[j + 4], v[j + 5]);
              o.w = pack_bf16x2(v[j + 6], v[j + 7]);
              *reinterpret_cast<uint4*>(srow + j * 2) = o;
            }
          }
        }
      }
      // accumulator drained: hand the TMEM buffer back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[acc]));
      if (p.epi_mode != RB_EPI_STORE) {
        // rows of this warp: q*32 .. q*32+31 of the tile; each row holds n_valid columns
        const int units_per_row = n_valid >> 3;                      // 16-byte units
        const int rows_here = min(32, (grp ? m_part : p.a_rows_per_part - m_in) - q * 32);
        const int n_dst = p.epi_mode == RB_EPI_ALL_REDUCE_ONESHOT ? p.world : 1;
        for (int u = lane; u < rows_here * units_per_row; u += 32) {
          const int rr = u / units_per_row, cu = u - rr * units_per_row;
          const uint4 o = *reinterpret_cast<const uint4*>(epi_stage + (size_t)rr * EPI_ROWB + cu * 16);
          const int r_in = m_in + q * 32 + rr;                         // row inside the A slab
          const int ccol = n_base + cu * 8;
          for (int di = 0; di < n_dst; ++di) {
            __nv_bfloat16* dst;
            if (p.epi_mode == RB_EPI_ALL_REDUCE_ONESHOT)
              dst = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<char*>(p.stage_ptrs[di]) + stage_off) +
                    ((long long)p.rank * p.M + (long long)m_part * p.a_rows_per_part + r_in) * p.N + ccol;
            else
              dst = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<char*>(p.stage_ptrs[m_part]) + stage_off) +
                    ((long long)p.rank * rows_per_rank + r_in) * p.N + ccol;
            *reinterpret_cast<uint4*>(dst) = o;
          }
        }
        __syncwarp();   // the slab is rewritten by the next tile
        // publish the tile: all 4 epilogue warps must have finished their peer stores
        RB_TS(2);
        __threadfence_system();
        RB_TS(3);
        ok = epi_sync();
        if (!ok) break;
        const int tile_in_part = (m_in / BM) * num_n_tiles + (n_part * n_tiles_per_part + n_in / BN);
        if (p.epi_mode == RB_EPI_ALL_REDUCE_ONESHOT) {
          if (warp == 2 && lane < p.world) {   // one flag per destination rank
            int* f = reinterpret_cast<int*>(reinterpret_cast<char*>(p.flag_ptrs[lane]) + flag_off) +
                     (long long)p.rank * (m_tiles_per_part * num_n_tiles) + tile_in_part;
            // every writer fenced at system scope before the barrier above: a relaxed store is enough and
            // saves the second fence round trip a release store would pay
            st_relaxed_sys(f, reduce_epoch);
          }
        } else if (warp == 2 && lane == 0) {
          int* f = reinterpret_cast<int*>(reinterpret_cast<char*>(p.flag_ptrs[m_part]) + flag_off) +
                   (long long)p.rank * (m_tiles_per_part * num_n_tiles) + tile_in_part;
          st_release_sys(f, reduce_epoch);
        }
      }
    }

    // ---------------- reduce phase: sum the P partials of the tiles this rank owns ----------
    if (p.epi_mode != RB_EPI_STORE && ok) {
      const int tiles_owned = m_tiles_per_part * num_n_tiles;
      const __nv_bfloat16* stage = reinterpret_cast<const __nv_bfloat16*>(reinterpret_cast<const char*>(p.stage_ptrs[p.rank]) + stage_off);
      const int* flags = reinterpret_cast<const int*>(reinterpret_cast<const char*>(p.flag_ptrs[p.rank]) + flag_off);
      const int et = (warp - 2) * 32 + lane;  // 0..127
      RB_TS(4);
      if (p.epi_mode == RB_EPI_ALL_REDUCE_ONESHOT) {
        // every rank holds all partials of every tile: sum the tiles this CTA computed, store locally
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
          int m_part, m_in, n_part, n_in, kb_lo_, kb_hi_;
          tile_coords(t, m_part, m_in, n_part, n_in, kb_lo_, kb_hi_);
          const int tile_idx = (m_in / BM) * num_n_tiles + (n_part * n_tiles_per_part + n_in / BN);
          if (et < p.world) {
            if (!wait_flag_ge(flags + (long long)et * tiles_owned + tile_idx, reduce_epoch, p.status)) *abortp = 1;
          }
          ok = epi_sync();
          RB_TS(5);
          if (!ok || *abortp) { ok = false; break; }
          const int n0 = n_part * p.b_rows_per_part + n_in;
          const int vec_per_row = min(BN, p.b_rows_per_part - n_in) / 8;
          const int rows = min(BM, p.M - m_in);
          // all loads of a batch are issued before the first add: the loop is a chain of L2 round trips otherwise
          constexpr int UNR = 4;
          const int total = rows * vec_per_row;
          for (int base = et; base < total; base += 128 * UNR) {
            uint4 part[UNR][8];
            uint4 res[UNR];
#pragma unroll
            for (int u = 0; u < UNR; ++u) {
              const int idx = base + u * 128;
              if (idx < total) {
                const long long row = m_in + idx / vec_per_row;
                const int col = n0 + (idx % vec_per_row) * 8;
#pragma unroll
                for (int src = 0; src < 8; ++src)
                  if (src < p.world)
                    part[u][src] = __ldcg(reinterpret_cast<const uint4*>(stage + ((long long)src * p.M + row) * p.N + col));
                if (p.residual != nullptr) res[u] = *reinterpret_cast<const uint4*>(p.residual + row * p.ldr + col);
              }
            }
#pragma unroll
            for (int u = 0; u < UNR; ++u) {
              const int idx = base + u * 128;
              if (idx >= total) break;
              const long long row = m_in + idx / vec_per_row;
              const int col = n0 + (idx % vec_per_row) * 8;
              float acc8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
              auto add = [&](const uint4& b) {
                float2 f;
                f = unpack_bf16x2(b.x); acc8[0] += f.x; acc8[1] += f.y;
                f = unpack_bf16x2(b.y); acc8[2] += f.x; acc8[3] += f.y;
                f = unpack_bf16x2(b.z); acc8[4] += f.x; acc8[5] += f.y;
                f = unpack_bf16x2(b.w); acc8[6] += f.x; acc8[7] += f.y;
              };
#pragma unroll
              for (int src = 0; src < 8; ++src)
                if (src < p.world) add(part[u][src]);
              if (p.bias != nullptr) {
#pragma unroll
                for (int j = 0; j < 8; ++j) acc8[j] += __bfloat162float(p.bias[col + j]);
              }
              if (p.residual != nullptr) add(res[u]);
              uint4 o;
              o.x = pack_bf16x2(acc8[0], acc8[1]);
              o.y = pack_bf16x2(acc8[2], acc8[3]);
              o.z = pack_bf16x2(acc8[4], acc8[5]);
              o.w = pack_bf16x2(acc8[6], acc8[7]);
              *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.C) + row * p.ldc + col) = o;
            }
          }
        }
      } else
      for (int ot = blockIdx.x; ot < tiles_owned && ok; ot += gridDim.x) {
        const int mt = ot / num_n_tiles, nt = ot % num_n_tiles;
        // wait for every source rank's copy of this tile
        if (et < p.world) {
          if (!wait_flag_ge(flags + (long long)et * tiles_owned + ot, reduce_epoch, p.status)) *abortp = 1;
        }
        ok = epi_sync();
        if (!ok || *abortp) { ok = false; break; }
        const int n_part = nt / n_tiles_per_part;
        const int n0 = n_part * p.b_rows_per_part + (nt % n_tiles_per_part) * BN;
        const int n_valid = min(BN, p.b_rows_per_part - (nt % n_tiles_per_part) * BN);
        const int m0 = mt * BM;
        const int vec_per_row = n_valid / 8;
        const int rows = min(BM, rows_per_rank - m0);
        // loads of two steps are in flight before the first add (each step reads `world` partial rows)
        constexpr int UNR2 = 2;
        const int total = rows * vec_per_row;
        for (int base = et; base < total; base += 128 * UNR2) {
          uint4 part[UNR2][8];   // up to 8 ranks (one NVLink domain); registers, not local memory
#pragma unroll
          for (int u = 0; u < UNR2; ++u) {
            const int idx = base + u * 128;
            if (idx < total) {
              const int row_in = m0 + idx / vec_per_row, col = n0 + (idx % vec_per_row) * 8;
#pragma unroll
              for (int src = 0; src < 8; ++src)
                if (src < p.world)
                  part[u][src] = __ldcg(reinterpret_cast<const uint4*>(stage + ((long long)src * rows_per_rank + row_in) * p.N + col));
            }
          }
#pragma unroll
          for (int u = 0; u < UNR2; ++u) {
            const int idx = base + u * 128;
            if (idx >= total) break;
            const int row_in = m0 + idx / vec_per_row, col = n0 + (idx % vec_per_row) * 8;
            float acc8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
            for (int src = 0; src < 8; ++src) {
              if (src < p.world) {
                const uint4 bq = part[u][src];
                float2 f;
                f = unpack_bf16x2(bq.x); acc8[0] += f.x; acc8[1] += f.y;
                f = unpack_bf16x2(bq.y); acc8[2] += f.x; acc8[3] += f.y;
                f = unpack_bf16x2(bq.z); acc8[4] += f.x; acc8[5] += f.y;
                f = unpack_bf16x2(bq.w); acc8[6] += f.x; acc8[7] += f.y;
              }
            }
            const long long grow = (long long)p.rank * rows_per_rank + row_in;
            if (p.bias != nullptr) {
#pragma unroll
              for (int j = 0; j < 8; ++j) acc8[j] += __bfloat162float(p.bias[col + j]);
            }
            if (p.residual != nullptr) {
              // reduce-scatter: residual is the local row slab; all-reduce: the full matrix
              const long long rrow = (p.epi_mode == RB_EPI_REDUCE_SCATTER) ? row_in : grow;
#pragma unroll
              for (int j = 0; j < 8; ++j) acc8[j] += __bfloat162float(p.residual[rrow * p.ldr + col + j]);
            }
            uint4 o;
            o.x = pack_bf16x2(acc8[0], acc8[1]);
            o.y = pack_bf16x2(acc8[2], acc8[3]);
            o.z = pack_bf16x2(acc8[4], acc8[5]);
            o.w = pack_bf16x2(acc8[6], acc8[7]);
            if (p.epi_mode == RB_EPI_REDUCE_SCATTER) {
              __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out_ptrs[p.rank]);
              *reinterpret_cast<uint4*>(out + (long long)row_in * p.ldc + col) = o;
            } else {
              for (int d = 0; d < p.world; ++d) {
                __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out_ptrs[d]);
                *reinterpret_cast<uint4*>(out + grow * p.ldc + col) = o;
              }
            }
          }
        }
      }
    }
    if (p.cluster_k && tile_iter > 0) {
      // peers may still be reading this CTA's last partial tile through distributed shared memory: stay
      // resident until they signalled, whatever else went wrong (only the time budget ends this wait)
      mbar_wait_bounded_cluster(smem_u32(&red_empty_bar), (tile_iter - 1) & 1u, abortp, p.status, ST_TIMEOUT_TMEM_EMPTY, false);
    }
  }

  RB_TS(6);
  // ------------------------------ teardown --------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  if (p.epoch_counter != nullptr && threadIdx.x == 0) {
    // every CTA read the counter before arriving here, so the last one may advance it
    __threadfence();
    if (atomicAdd(p.cta_ticket, 1) == (int)gridDim.x - 1) {
      *p.cta_ticket = 0;
      *p.epoch_counter = reduce_epoch;
      __threadfence();
    }
  }
}

// ---------------------------------- host side ------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(f);
    }
  });
  return fn;
}

// 2-D bf16 tensor map over `rows` x `cols` (cols contiguous, leading dimension ld elements),
// box = box_rows x 64 columns, 128-byte swizzle.
static int make_map_2d(CUtensorMap* out, const void* base, long long rows, long long cols,
                       long long ld, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (ld * 2) % 16 != 0) return -2;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

static int num_sms() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

#ifdef RB_GEMM_TIMESTAMPS
}  // namespace rb
extern "C" int rb_gemm_read_timestamps(unsigned long long* out, int n) {
  return cudaMemcpyFromSymbol(out, rb::g_ts, sizeof(unsigned long long) * n) == cudaSuccess ? 0 : -1;
}
namespace rb {
#endif

constexpr int kMaxDynSmem = 227 * 1024 - 2048;   // 227 KB per CTA minus the kernel's static shared memory (about 1.3 KB)

template <int BN, bool A_MN, bool B_MN, bool NORM = false, bool GATHER = false>
static int launch_cfg(const GemmParams& p, int max_ctas, cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, NORM, GATHER>;
  static bool attr_dev[64] = {};       // the shared-memory opt-in is a per-device function attribute
  int dev_i = 0;
  if (cudaGetDevice(&dev_i) != cudaSuccess || dev_i < 0 || dev_i >= 64) return -10;
  bool& attr_set = attr_dev[dev_i];
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynSmem);
    if (e != cudaSuccess) return -10;
    attr_set = true;
  }
  const int m_tiles = ((p.a_rows_per_part + BM - 1) / BM) * p.a_parts;
  const int n_tiles = ((p.b_rows_per_part + BN - 1) / BN) * p.b_parts;
  int grid = m_tiles * n_tiles * (p.split_k > 1 ? p.split_k : 1);
  if (p.tile_table != nullptr) grid = max_ctas > 0 ? max_ctas : num_sms();  // tile count is only known on the device
  int cap = num_sms();
  if (max_ctas > 0 && max_ctas < cap) cap = max_ctas;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  if (p.cluster_k) {
    grid -= grid % p.split_k;                       // whole clusters only
    if (grid < p.split_k || BN / p.split_k < 8) return -15;
  }
  // Ring depth: never deeper than the k-blocks a CTA will load in total.
  GemmParams q = p;
  int stages = Cfg::kStages;
  if (p.tile_table == nullptr) {
    const long long units = (long long)m_tiles * n_tiles * (p.split_k > 1 ? p.split_k : 1);
    const long long units_per_cta = (units + grid - 1) / grid;
    const int num_kb = (p.K + BK - 1) / BK;
    const long long kb_cta = units_per_cta * (p.split_k > 1 ? p.kb_per_split : num_kb);
    if (kb_cta < stages) stages = kb_cta < 2 ? 2 : (int)kb_cta;
  }
  // reduce modes stage the outgoing partial tile in shared memory behind the ring
  // cluster split-K parks the fp32 partial tile ([BN/4 column quads][BM rows] float4) there instead; with one
  // unit per CTA the partial reuses the ring itself
  int extra = p.cluster_k ? BM * BN * 4 : p.epi_mode != RB_EPI_STORE ? 128 * (BN * 2 + 16) : 0;
  if (p.cluster_k) {
    const long long units = (long long)m_tiles * n_tiles * p.split_k;
    q.red_alias = units <= grid ? 1 : 0;
  }
  int fit = (kMaxDynSmem - 1024 - (q.red_alias ? 0 : extra)) / Cfg::kStageBytes;
  if (stages > fit) stages = fit;
  if (stages < 2) return -14;
  q.stages = stages;
  int smem = stages * Cfg::kStageBytes + 1024 + extra;
  if (q.red_alias) smem = (stages * Cfg::kStageBytes > extra ? stages * Cfg::kStageBytes : extra) + 1024;
  if (p.cluster_k)
    return launch_kernel_cluster(kern, dim3(grid), dim3(GEMM_THREADS), smem, stream, (unsigned)p.split_k, q) == cudaSuccess ? 0 : -11;
  return launch_kernel(kern, dim3(grid), dim3(NORM ? GEMM_THREADS_NORM : (GATHER ? GEMM_THREADS_GATHER : GEMM_THREADS)), smem,
                       stream, q) == cudaSuccess ? 0 : -11;
}

template <int BN>
static int launch_bn(const GemmParams& p, int a_mn, int b_mn, int max_ctas, cudaStream_t s) {
  if (p.gather_parts > 0) {
    // launches that carry an all-gather: forward (K-major operands) and weight gradient (both MN-major), wide tiles
    if (!a_mn && !b_mn) return launch_cfg<BN, false, false, false, true>(p, max_ctas, s);
    if constexpr (BN >= 128) {
      if (a_mn && b_mn) return launch_cfg<BN, true, true, false, true>(p, max_ctas, s);
    }
    return -12;
  }
  if (!a_mn && !b_mn) return p.norm_fold ? launch_cfg<BN, false, false, true>(p, max_ctas, s) : launch_cfg<BN, false, false>(p, max_ctas, s);
  if (p.norm_fold) return -12;   // the folded norm exists for K-major operands only
  if constexpr (BN >= 64) {
    if (!a_mn && b_mn) return launch_cfg<BN, false, true>(p, max_ctas, s);
    if (a_mn && b_mn) return launch_cfg<BN, true, true>(p, max_ctas, s);
  }
  if (a_mn && !b_mn) return launch_cfg<BN, true, false>(p, max_ctas, s);
  return -12;
}

// Tile-width choice. A persistent CTA streams its tiles one after another, so the launch
// costs waves x (fixed + k-blocks x stage bytes / per-SM streaming rate); e.g. 152 tiles on 148
// SMs cost two full waves, which a wider tile avoids.
static int pick_bn(int m_tiles, int n_rows_per_part, int parts, int b_mn, int K) {
  const int sms = num_sms();
  const int cands[4] = {256, 128, 64, 32};
  const double num_kb = (K + BK - 1) / BK;
  int best = b_mn ? 64 : 32;
  double best_cost = 1e30;
  for (int i = 0; i < 4; ++i) {
    const int bn = cands[i];
    if (b_mn && bn < 64) continue;
    const int tiles = m_tiles * ((n_rows_per_part + bn - 1) / bn) * parts;
    const double waves = (tiles + sms - 1) / sms;
    const double stage_us = (double)(BM + bn) * BK * 2 / 100e3;   // ~100 GB/s per SM
    const double mma_us = (double)BM * bn * BK * 2 / 8.0e6;        // ~8 TFLOP/s per SM
    const double per_tile = 2.5 + num_kb * (stage_us > mma_us ? stage_us : mma_us);
    const double cost = waves * per_tile;
    if (cost < best_cost * 0.98) { best_cost = cost; best = bn; }
  }
  return best;
}

}  // namespace rb

using namespace rb;

extern "C" int rb_gemm_bf16_ex(const RbGemmArgs* a, cudaStream_t stream) {
  if (a == nullptr) return -1;
  if (a->M <= 0 || a->N <= 0 || a->K <= 0) return -1;
  if (a->a_parts < 1 || a->a_parts > RB_MAX_PARTS || a->b_parts < 1 || a->b_parts > RB_MAX_PARTS) return -1;
  if (a->M % a->a_parts != 0 || a->N % a->b_parts != 0) return -1;
  if (a->N % 8 != 0) return -1;
  // K is a row stride only for K-major operands; MN-major operands may have any K (TMA zero-fills)
  if ((!a->a_mn_major || !a->b_mn_major) && a->K % 8 != 0) return -1;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = a->M; p.N = a->N; p.K = a->K;
  p.a_parts = a->a_parts; p.b_parts = a->b_parts;
  p.a_rows_per_part = a->M / a->a_parts;
  p.b_rows_per_part = a->N / a->b_parts;
  if (p.b_rows_per_part % 8 != 0) return -1;
  p.C = a->C; p.ldc = a->ldc;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(a->bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(a->residual);
  p.ldr = a->ldr;
  p.out_f32 = a->out_f32;
  p.epi_mode = a->epi_mode;
  p.a_ready = a->a_ready; p.b_ready = a->b_ready; p.ready_epoch = a->ready_epoch;
  p.ready_epoch_ptr = a->ready_epoch_ptr;
  p.rank = a->rank; p.world = a->world < 1 ? 1 : a->world;
  p.reduce_epoch = a->reduce_epoch;
  p.status = a->status;
  p.epoch_counter = a->epoch_counter;
  p.cta_ticket = a->cta_ticket;
  p.stage_parity_bytes = a->stage_parity_bytes;
  p.flag_parity_bytes = a->flag_parity_bytes;
  if (p.epoch_counter != nullptr && p.cta_ticket == nullptr) return -1;
  p.tile_table = reinterpret_cast<const int4*>(a->tile_table);
  p.num_tiles_ptr = a->num_tiles_ptr;
  p.row_dst = a->row_dst;
  p.swiglu = a->swiglu;
  p.scaled_epilogue = a->scaled_epilogue;
  p.alpha = a->alpha;
  p.beta = a->beta;
  p.mirror = a->mirror;
  p.fp8 = a->fp8;
  p.sample_ws = a->sample_ws;
  p.sample_temperature = a->sample_temperature;
  p.sample_seeds = a->sample_seeds;
  p.sample_step_ptr = a->sample_step_ptr;
  p.sample_step_add = a->sample_step_add;
  if (p.sample_ws != nullptr && (a->tile_table || a->swiglu || a->split_k > 1 || a->epi_mode != RB_EPI_STORE || a->a_parts != 1 ||
                                a->b_parts != 1 || !a->sample_temperature || !a->sample_seeds))
    return -1;
  if (p.fp8 && (a->a_mn_major || a->b_mn_major)) return -1;   // 8-bit operands are K-major only
  p.split_k = a->split_k > 1 ? a->split_k : 1;
  p.splitk_ws = a->splitk_ws;
  p.splitk_tickets = a->splitk_tickets;
  p.kb_per_split = 0;
  p.norm_fold = a->norm_fold ? 1 : 0;
  p.norm_eps = a->norm_eps;
  p.norm_inv_k = 1.f / (float)a->K;
  if (p.norm_fold && (a->a_mn_major || a->split_k > 1 || a->epi_mode != RB_EPI_STORE || a->tile_table || p.sample_ws != nullptr ||
                      a->a_parts != 1 || p.fp8 || p.mirror || a->row_dst))
    return -1;
  if (a->gather_parts > 0) {
    if (a->gather_parts > RB_MAX_PARTS || a->gather_dst == nullptr || a->gather_count == nullptr || a->gather_ready == nullptr ||
        a->gather_part_bytes <= 0 || a->gather_part_bytes % 16 != 0 || p.norm_fold || a->split_k > 1 || a->tile_table ||
        a->swiglu || p.epi_mode != RB_EPI_STORE || p.sample_ws != nullptr || a->rank < 0 || a->rank >= a->gather_parts)
      return -1;
    p.gather_parts = a->gather_parts;
    for (int r = 0; r < a->gather_parts; ++r) p.gather_src[r] = a->gather_src[r];
    p.gather_dst = a->gather_dst;
    p.gather_part_bytes = a->gather_part_bytes;
    p.gather_count = a->gather_count;
    p.gather_ready = a->gather_ready;
    p.gather_epoch = a->gather_epoch;
    p.gather_src_ready = a->gather_src_ready;
    p.gather_wait_all = a->gather_wait_all ? 1 : 0;
  }
  p.b_part_rot = (a->b_part_rot > 0 && a->b_part_rot < a->b_parts) ? a->b_part_rot : 0;
  p.cluster_k = (a->cluster_split && p.split_k > 1) ? 1 : 0;
  if (p.cluster_k) {
    // slices = CTAs of one cluster; needs a power-of-two slice count up to 8 and a non-empty K range for each
    const int S = p.split_k, num_kb = (a->K + BK - 1) / BK;
    if ((S != 2 && S != 4 && S != 8) || a->swiglu || a->tile_table || p.epi_mode != RB_EPI_STORE || a->a_parts != 1 ||
        a->b_parts != 1 || p.sample_ws != nullptr || p.scaled_epilogue || p.mirror)
      return -1;
    p.kb_per_split = (num_kb + S - 1) / S;
    if ((S - 1) * p.kb_per_split >= num_kb) return -1;
  } else if (p.split_k > 1) {
    if (p.splitk_ws == nullptr || p.splitk_tickets == nullptr || a->swiglu || a->tile_table || p.epi_mode != RB_EPI_STORE ||
        a->a_parts != 1 || a->b_parts != 1 || a->N % 4 != 0)
      return -1;
    const int num_kb = (a->K + BK - 1) / BK;
    p.kb_per_split = (num_kb + p.split_k - 1) / p.split_k;
    p.split_k = (num_kb + p.kb_per_split - 1) / p.kb_per_split;  // no empty slices
    if (p.split_k <= 1) { p.split_k = 1; p.kb_per_split = 0; }
  }
  if (p.swiglu) {
    if (a->bn < 64 || a->N % a->bn != 0 || a->b_parts != 1 || a->out_f32 || p.epi_mode != RB_EPI_STORE || a->bias ||
        a->residual || a->tile_table)
      return -1;
  }
  if (p.tile_table != nullptr) {
    if (p.num_tiles_ptr == nullptr || a->group_n <= 0 || a->group_n % 8 != 0 || a->a_parts != 1 || a->b_parts != 1 ||
        a->bn == 0 || p.epi_mode != RB_EPI_STORE)
      return -1;
    const int gm = a->group_mode;
    if (gm == 0 ? (a->a_mn_major || a->b_mn_major)
        : gm == 1 ? (a->a_mn_major || !a->b_mn_major || a->group_b_rows <= 0 || a->K % BK != 0 || a->row_dst || a->swiglu)
        : gm == 2 ? (!a->a_mn_major || !a->b_mn_major || a->K % BK != 0 || a->row_dst || a->swiglu || a->bn < 64)
                  : true)
      return -1;
    p.group_k = gm == 2;
  } else if (a->group_mode != 0) {
    return -1;
  }
  if (p.epi_mode != RB_EPI_STORE) {
    if (p.epi_mode == RB_EPI_ALL_REDUCE_ONESHOT ? (a->a_parts != 1 || a->b_parts != 1) : (a->a_parts != p.world)) return -1;
    if (a->out_f32 || p.world > 8) return -1;   // the reduce keeps one partial per rank in registers
    if (p.a_rows_per_part % 8 != 0) return -1;
    for (int r = 0; r < p.world; ++r) {
      p.stage_ptrs[r] = a->stage_ptrs[r];
      p.flag_ptrs[r] = a->flag_ptrs[r];
      p.out_ptrs[r] = a->out_ptrs[r];
    }
  }
  const int m_tiles = ((p.a_rows_per_part + BM - 1) / BM) * p.a_parts;
  const int total_b_rows = p.b_rows_per_part;   // rows of the (stacked) B matrix for its tensor map
  if (p.tile_table != nullptr) p.b_rows_per_part = a->group_n;  // columns valid per group
  int bn = a->bn;
  if (bn == 0) {
    bn = pick_bn(m_tiles, p.b_rows_per_part, p.b_parts, a->b_mn_major, p.K);
    // partial tiles cross NVLink row by row: at least 128 contiguous bytes per row
    if (p.epi_mode != RB_EPI_STORE && bn < 64) bn = 64;
  }
  if (a->b_mn_major && bn < 64) bn = 64;
  if (p.gather_parts > 0 && bn < 128 && !p.gather_wait_all) bn = 128;   // weight gathers ride on wide-tile launches
  // tensor maps: one per slab
  for (int i = 0; i < p.a_parts; ++i) {
    int rc = a->a_mn_major
                 ? make_map_2d(&p.a_map[i], a->A[i], a->K, p.a_rows_per_part, a->lda, BK)
                 : make_map_2d(&p.a_map[i], a->A[i], p.a_rows_per_part, a->K, a->lda, BM);
    if (rc != 0) return -20 + rc;
  }
  for (int i = 0; i < p.b_parts; ++i) {
    int rc = a->b_mn_major
                 ? make_map_2d(&p.b_map[i], a->B[i], a->group_mode == 1 ? a->group_b_rows : a->K, total_b_rows, a->ldb, BK)
                 : make_map_2d(&p.b_map[i], a->B[i], total_b_rows, a->K, a->ldb, bn);
    if (rc != 0) return -30 + rc;
  }
  switch (bn) {
    case 32: return launch_bn<32>(p, a->a_mn_major, a->b_mn_major, a->max_ctas, stream);
    case 64: return launch_bn<64>(p, a->a_mn_major, a->b_mn_major, a->max_ctas, stream);
    case 128: return launch_bn<128>(p, a->a_mn_major, a->b_mn_major, a->max_ctas, stream);
    case 256: return launch_bn<256>(p, a->a_mn_major, a->b_mn_major, a->max_ctas, stream);
    default: return -13;
  }
}

namespace rb {
__global__ void sample_merge_kernel(const float4* __restrict__ ws, int M, int n_tiles, int* __restrict__ out_tokens,
                                    float* __restrict__ out_logprobs) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= M) return;
  float m = -INFINITY, ssum = 0.f, best = -INFINITY, best_logit = 0.f;
  int best_i = 0x7fffffff;
  for (int t = lane; t < n_tiles; t += 32) {
    const float4 a = ws[((long long)row * n_tiles + t) * 2], b = ws[((long long)row * n_tiles + t) * 2 + 1];
    const float mn = fmaxf(m, a.x);
    ssum = (mn == -INFINITY) ? 0.f : ssum * __expf(m - mn) + a.y * __expf(a.x - mn);
    m = mn;
    const int bi = __float_as_int(b.x);
    if (a.z > best || (a.z == best && bi < best_i)) { best = a.z; best_i = bi; best_logit = a.w; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, ssum, o);
    const float b2 = __shfl_xor_sync(0xffffffffu, best, o), l2 = __shfl_xor_sync(0xffffffffu, best_logit, o);
    const int i2 = __shfl_xor_sync(0xffffffffu, best_i, o);
    const float mn = fmaxf(m, m2);
    ssum = (mn == -INFINITY) ? 0.f : ssum * __expf(m - mn) + s2 * __expf(m2 - mn);
    m = mn;
    if (b2 > best || (b2 == best && i2 < best_i)) { best = b2; best_i = i2; best_logit = l2; }
  }
  if (lane == 0) {
    out_tokens[row] = best_i;
    out_logprobs[row] = best_logit - (m + __logf(ssum));
  }
}
}  // namespace rb

extern "C" int rb_sample_merge(const float* sample_ws, int M, int n_tiles, int* out_tokens, float* out_logprobs,
                               cudaStream_t stream) {
  if (M <= 0) return 0;
  return rb::launch_kernel(rb::sample_merge_kernel, dim3((M + 3) / 4), dim3(128), 0, stream,
                           reinterpret_cast<const float4*>(sample_ws), M, n_tiles, out_tokens, out_logprobs) == cudaSuccess ? 0 : -11;
}

extern "C" void rb_gemm_set_pdl(int on) { rb::pdl_enabled() = on != 0; }

// Plain single-GPU form: C = A * B^T (+bias) (+residual).
extern "C" int rb_gemm_bf16(const void* A, const void* B, void* C, const void* bias,
                            const void* residual, int M, int N, int K, long long lda,
                            long long ldb, long long ldc, long long ldr, int a_mn_major,
                            int b_mn_major, int out_f32, int bn, int* status,
                            cudaStream_t stream) {
  RbGemmArgs a;
  memset(&a, 0, sizeof(a));
  a.A[0] = A; a.B[0] = B; a.C = C; a.bias = bias; a.residual = residual;
  a.M = M; a.N = N; a.K = K; a.lda = lda; a.ldb = ldb; a.ldc = ldc; a.ldr = ldr;
  a.a_parts = 1; a.b_parts = 1;
  a.a_mn_major = a_mn_major; a.b_mn_major = b_mn_major; a.out_f32 = out_f32; a.bn = bn;
  a.epi_mode = RB_EPI_STORE; a.world = 1; a.status = status;
  return rb_gemm_bf16_ex(&a, stream);
}
