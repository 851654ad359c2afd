// Two-CTA bf16 GEMM for sm_100a: one 256 x BN output tile per pair of CTAs (a thread-block cluster of two),
// computed by `tcgen05.mma.cta_group::2`.
//
//   C[M,N] = op(A) * op(B)^T (+ bias) (+ residual)      fp32 accumulate in TMEM, bf16 or fp32 output
//
// Why a second GEMM kernel: the one-CTA kernel (gemm_sm100.cu) stages 128 x 64 of A and BN x 64 of B per k-block
// in every SM, and what bounds it on large problems is the shared-memory traffic of those operand tiles. With the
// pair instruction each CTA stages its own 128 rows of A but only HALF of the B tile (BN/2 rows): the tensor cores
// of both SMs read both halves. Per SM that is one third fewer operand bytes per FLOP at BN = 256, which is the
// difference between about 0.8 and the library's throughput on the training shapes.
//
// Layout of a pair (cluster ranks 0 = leader, 1 = peer), tile rows m0 .. m0+255, columns n0 .. n0+BN-1:
//   * CTA r loads A rows m0 + 128 r .. +127 and B rows n0 + (BN/2) r .. into ITS shared memory with plain
//     (non-broadcast) TMA tile loads; every load of both CTAs signals the LEADER's "full" mbarrier of that stage;
//   * one thread of the leader issues the MMAs (M = 256, N = BN, K = 16) for both SMs and commits them to the
//     "empty" mbarrier of the stage in both CTAs and, after the last k-block, to the "accumulator full" mbarrier
//     of both CTAs;
//   * each CTA's four epilogue warps drain its own 128 TMEM lanes (all BN columns of its 128 rows) and arrive on
//     the leader's "accumulator empty" mbarrier; the accumulator is double buffered (2 x BN columns).
// Operand majorness is a descriptor flag as in the one-CTA kernel, so forward (K-major, K-major), dgrad
// (K-major, MN-major) and wgrad (MN-major, MN-major) run on the same code. Every wait is bounded; a CTA that gives
// up drains its copies, meets its peer at the cluster barrier and frees its TMEM before it returns.
#include "common.cuh"
#include "tma_host.h"

#include <string.h>

namespace rb {

constexpr int G2_BM = 128;            // rows of A per CTA (256 per pair)
constexpr int G2_BK = 64;
constexpr int G2_THREADS = 192;       // warp 0 TMA, warp 1 TMEM + MMA, warps 2-5 epilogue
constexpr int G2_EPI_WARPS = 4;
constexpr int G2_ACC = 2;

template <int BN>
struct G2Cfg {
  static constexpr int kABytes = G2_BM * G2_BK * 2;            // 16 KB
  static constexpr int kBBytes = (BN / 2) * G2_BK * 2;         // this CTA's half of the B tile
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN == 256) ? 6 : 8;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024;
  static constexpr int kTmemCols = G2_ACC * BN;               // 512 or 256
};

struct G2Params {
  CUtensorMap a_map, b_map;
  int M, N, K;
  void* C;
  long long ldc;
  const __nv_bfloat16* residual;
  long long ldr;
  const __nv_bfloat16* bias;
  int out_f32;
  int* status;
  // Fused all-gather of a row-sharded matrix (GATHER instantiations; same contract as the one-CTA kernel): part r is
  // gather_part_bytes at gather_src[r] (rank r's shard, peer memory); the gather warps of every CTA copy an
  // interleaved share of each part to gather_dst + r * bytes, own part first, and the last CTA to finish a part
  // publishes gather_ready[r] = gather_epoch. With `consume` the gathered matrix is this launch's K-major B operand:
  // tiles visit the parts starting at the local one and their producers wait for the part they read.
  const void* gather_src[8];
  void* gather_dst;
  long long gather_part_bytes;
  int* gather_count;
  int* gather_ready;
  int gather_epoch, gather_parts, rank, consume, n_tiles_per_part;
  // A part is copied and published in `gather_chunks` pieces of gather_chunk_tiles column tiles (256 rows of the
  // gathered matrix) each, so the tiles of a remote part start while the rest of it is still crossing NVLink:
  // flag / counter index = part * gather_chunks + chunk.
  int gather_chunks, gather_chunk_tiles;
  long long gather_chunk_bytes;
};
constexpr int G2_GATHER_WARPS = 4;      // measured with 2: the copy (159 GB/s over NVLink) set the launch's time
constexpr int G2_THREADS_GATHER = G2_THREADS + 32 * G2_GATHER_WARPS;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Tile load whose completion may be signalled on an mbarrier of either CTA of the pair (no broadcast: the data lands
// in the issuing CTA's shared memory only).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma2_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The mbarrier (an address in the cluster's shared window: this CTA's or the peer's) receives one arrival once every
// tcgen05 operation issued so far by this thread has completed in both CTAs.
__device__ __forceinline__ void umma2_commit(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}

template <int BN, bool A_MN, bool B_MN, bool GATHER = false>
__global__ void __launch_bounds__(GATHER ? G2_THREADS_GATHER : G2_THREADS, 1) gemm2cta_kernel(const __grid_constant__ G2Params p) {
  using Cfg = G2Cfg<BN>;
  constexpr int STAGES = Cfg::kStages;
  constexpr int HALF_N = BN / 2;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[STAGES];       // used in the leader: both CTAs' loads of the stage landed
  __shared__ __align__(8) uint64_t empty_bar[STAGES];      // per CTA: the MMAs that read the stage have retired
  __shared__ __align__(8) uint64_t tmem_full_bar[G2_ACC];  // per CTA: the accumulator is complete
  __shared__ __align__(8) uint64_t tmem_empty_bar[G2_ACC]; // used in the leader: both CTAs' epilogues drained it
  __shared__ uint32_t tmem_base_smem;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();          // 0 = leader, 1 = peer
  const bool leader = cta == 0;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int m_tiles = (p.M + 255) / 256, n_tiles = (p.N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;
  const int num_kb = (p.K + G2_BK - 1) / G2_BK;
  // tile t -> (row tile, column tile); a launch that consumes its own gather starts at the local part's columns
  const int nt_rot = (GATHER && p.consume) ? p.rank * p.n_tiles_per_part : 0;
  auto tile_mn = [&](int t, int& mt, int& nt) {
    mt = t % m_tiles;
    nt = t / m_tiles + nt_rot;
    if (nt >= n_tiles) nt -= n_tiles;
  };

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < G2_ACC; ++a) {
      mbar_init(smem_u32(&tmem_full_bar[a]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[a]), 2 * G2_EPI_WARPS);
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_smem), Cfg::kTmemCols);   // the only allocation of this CTA: both CTAs get the same columns
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  cluster_sync_all();    // the peer's barriers exist before anything signals them
  const uint32_t tmem_base = tmem_base_smem;
  volatile int* abortp = &abort_flag;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) -----------------------------------
    if (elect_one_sync()) {
      int s = 0;
      uint32_t ph = 0, issued = 0;
      bool ok = true;
      unsigned long long chunks_seen = 0;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        int mt, nt;
        tile_mn(t, mt, nt);
        const int m0 = mt * 256 + (int)cta * G2_BM;        // this CTA's rows of A
        const int n0 = nt * BN + (int)cta * HALF_N;        // this CTA's rows of B
        if (GATHER && p.consume) {
          const int part = nt / p.n_tiles_per_part;
          const int idx = part * p.gather_chunks + (nt - part * p.n_tiles_per_part) / p.gather_chunk_tiles;
          if (!((chunks_seen >> idx) & 1ull)) {
            ok = wait_flag_ge(p.gather_ready + idx, p.gather_epoch, p.status);
            if (!ok) { *abortp = 1; break; }
            // the rows were written by ordinary stores of the gather warps: order them before the async-proxy tile loads
            asm volatile("fence.proxy.async.global;" ::: "memory");
            chunks_seen |= 1ull << idx;
          }
        }
        for (int kb = 0; kb < num_kb; ++kb, ++issued) {
          ok = mbar_wait_bounded_cluster(smem_u32(&empty_bar[s]), ph ^ 1u, abortp, p.status, ST_TIMEOUT_SMEM_EMPTY);
          if (!ok) break;
          const uint32_t fb = mapa_cluster(smem_u32(&full_bar[s]), 0);       // the leader's barrier of this stage
          if (leader) mbar_expect_tx(smem_u32(&full_bar[s]), 2 * Cfg::kStageBytes);
          const uint32_t sa = smem_base + s * Cfg::kStageBytes, sb = sa + Cfg::kABytes;
          if (!A_MN) {
            tma_load_2d_pair(sa, &p.a_map, fb, kb * G2_BK, m0);
          } else {
#pragma unroll
            for (int c = 0; c < G2_BM / 64; ++c) tma_load_2d_pair(sa + c * (G2_BK * 128), &p.a_map, fb, m0 + c * 64, kb * G2_BK);
          }
          if (!B_MN) {
            tma_load_2d_pair(sb, &p.b_map, fb, kb * G2_BK, n0);
          } else {
#pragma unroll
            for (int c = 0; c < HALF_N / 64; ++c) tma_load_2d_pair(sb + c * (G2_BK * 128), &p.b_map, fb, n0 + c * 64, kb * G2_BK);
          }
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
      }
      if (!ok) {
        // never leave with bulk copies still landing in this CTA's shared memory: the stage of copy j is free again
        // only after its data arrived, so give the copies in flight a moment (nothing else can be observed from the
        // peer's side, whose barrier they signal)
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 20000ull) { }
      }
      (void)issued;
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader only) ------------------------------------
    if (leader && elect_one_sync()) {
      constexpr uint32_t idesc = make_idesc_bf16(256, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int s = 0;
      uint32_t ph = 0, tile_iter = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs, ++tile_iter) {
        const int acc = tile_iter % G2_ACC;
        const uint32_t acc_ph = (tile_iter / G2_ACC) & 1u;
        ok = mbar_wait_bounded_cluster(smem_u32(&tmem_empty_bar[acc]), acc_ph ^ 1u, abortp, p.status, ST_TIMEOUT_TMEM_EMPTY);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait_bounded_cluster(smem_u32(&full_bar[s]), ph, abortp, p.status, ST_TIMEOUT_SMEM_FULL);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_base + s * Cfg::kStageBytes, sb = sa + Cfg::kABytes;
#pragma unroll
          for (int k = 0; k < G2_BK / 16; ++k) {
            const uint64_t adesc = A_MN ? make_smem_desc_sw128(sa + k * 2048, G2_BK * 128, 1024)
                                        : make_smem_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc_sw128(sb + k * 2048, G2_BK * 128, 1024)
                                        : make_smem_desc_sw128(sb + k * 32, 16, 1024);
            umma2_bf16(tmem_d, adesc, bdesc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          // the stage is free in BOTH CTAs once these MMAs retire
          umma2_commit(mapa_cluster(smem_u32(&empty_bar[s]), 0));
          umma2_commit(mapa_cluster(smem_u32(&empty_bar[s]), 1));
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        if (ok) {
          umma2_commit(mapa_cluster(smem_u32(&tmem_full_bar[acc]), 0));
          umma2_commit(mapa_cluster(smem_u32(&tmem_full_bar[acc]), 1));
        }
      }
    }
  } else if (GATHER && warp >= 2 + G2_EPI_WARPS) {
    // ------------------------------ gather warps (both CTAs) ------------------------------------
    constexpr int GT = 32 * G2_GATHER_WARPS;
    const int gt = (warp - 2 - G2_EPI_WARPS) * 32 + lane;
    const long long stride = (long long)gridDim.x * GT;
    for (int pp = 0; pp < p.gather_parts; ++pp) {
      int part = p.rank + pp;
      if (part >= p.gather_parts) part -= p.gather_parts;
      for (int ch = 0; ch < p.gather_chunks; ++ch) {
        const long long b0 = (long long)ch * p.gather_chunk_bytes;
        const long long b1 = min(b0 + p.gather_chunk_bytes, p.gather_part_bytes);
        const long long nvec = (b1 - b0) >> 4;
        const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(p.gather_src[part]) + b0);
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<char*>(p.gather_dst) + (long long)part * p.gather_part_bytes + b0);
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
          const int idx = part * p.gather_chunks + ch;
          const int old = atomicAdd(p.gather_count + idx, 1);
          if (old == (int)gridDim.x - 1) {     // every CTA's share of these rows is in place
            p.gather_count[idx] = 0;
            __threadfence();
            st_release_sys(p.gather_ready + idx, p.gather_epoch);
          }
        }
      }
    }
  } else {
    // ------------------------------ epilogue warps (both CTAs) ----------------------------------
    const int q = warp & 3;                       // TMEM lane quarter this warp may access
    uint32_t tile_iter = 0;
    bool ok = true;
    const uint32_t leader_empty0 = mapa_cluster(smem_u32(&tmem_empty_bar[0]), 0);
    const uint32_t leader_empty1 = mapa_cluster(smem_u32(&tmem_empty_bar[1]), 0);
    for (int t = pair; t < num_tiles && ok; t += num_pairs, ++tile_iter) {
      int mt, nt;
      tile_mn(t, mt, nt);
      const int acc = tile_iter % G2_ACC;
      const uint32_t acc_ph = (tile_iter / G2_ACC) & 1u;
      ok = mbar_wait_bounded_cluster(smem_u32(&tmem_full_bar[acc]), acc_ph, abortp, p.status, ST_TIMEOUT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
      const long long row = (long long)mt * 256 + (long long)cta * G2_BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      const int n_base = nt * BN;
      const int n_valid = min(BN, p.N - n_base);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + acc * BN + c0 + ((uint32_t)(q * 32) << 16), r);
        tmem_ld_wait();
        const int ncols = min(32, n_valid - c0);
        if (row_ok && ncols > 0) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          const int col = n_base + c0;
          if (p.bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (j < ncols) {
                const uint4 b = *reinterpret_cast<const uint4*>(p.bias + col + j);
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
                const uint4 b = *reinterpret_cast<const uint4*>(rp + j);
                float2 f;
                f = unpack_bf16x2(b.x); v[j] += f.x; v[j + 1] += f.y;
                f = unpack_bf16x2(b.y); v[j + 2] += f.x; v[j + 3] += f.y;
                f = unpack_bf16x2(b.z); v[j + 4] += f.x; v[j + 5] += f.y;
                f = unpack_bf16x2(b.w); v[j + 6] += f.x; v[j + 7] += f.y;
              }
            }
          }
          if (p.out_f32) {
            float* dst = reinterpret_cast<float*>(p.C) + row * p.ldc + col;
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              if (j < ncols) *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
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
      }
      // accumulator drained in this CTA: tell the leader's MMA thread
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc == 0 ? leader_empty0 : leader_empty1);
    }
  }

  // ------------------------------ teardown ------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();      // no CTA leaves while its peer may still signal one of its barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ---------------------------------- host side ------------------------------------------------
template <int BN, bool A_MN, bool B_MN, bool GATHER = false>
static int g2_launch(const G2Params& p, int tiles, cudaStream_t stream) {
  using Cfg = G2Cfg<BN>;
  auto kern = gemm2cta_kernel<BN, A_MN, B_MN, GATHER>;
  constexpr int THREADS = GATHER ? G2_THREADS_GATHER : G2_THREADS;
  static bool attr_set[64] = {};
  static int max_pairs[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -10;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess) return -10;
    int sms = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // how many pairs the device can hold at once (a persistent grid larger than that would only queue)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sms - sms % 2);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1) { cudaGetLastError(); n = sms / 2; }
    max_pairs[dev] = n < sms / 2 ? n : sms / 2;
    attr_set[dev] = true;
  }
  int pairs = tiles < max_pairs[dev] ? tiles : max_pairs[dev];
  if (GATHER) pairs = max_pairs[dev];      // every resident CTA copies a share of the gather, whatever the tile count
  if (pairs < 1) pairs = 1;
  return launch_kernel_cluster(kern, dim3(2 * pairs), dim3(THREADS), Cfg::kSmemBytes, stream, 2u, p) == cudaSuccess ? 0 : -11;
}

}  // namespace rb

using namespace rb;

// Number of CTA pairs a launch of width `bn` keeps resident (for the caller's choice of tile width).
extern "C" int rb_gemm2_pairs() {
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms / 2;
}

// C[M,N] = op(A) op(B)^T (+bias) (+residual). K-major operands are [rows, K] with K contiguous, MN-major operands
// [K, rows] with rows contiguous (as in rb_gemm_bf16). bn: 256 or 128 output columns per tile (0 = choose).
extern "C" int rb_gemm2_bf16(const void* A, const void* B, void* C, const void* bias, const void* residual, int M, int N,
                             int K, long long lda, long long ldb, long long ldc, long long ldr, int a_mn_major,
                             int b_mn_major, int out_f32, int bn, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || N % 8 != 0) return -1;
  if ((!a_mn_major || !b_mn_major) && K % 8 != 0) return -1;
  if (a_mn_major && !b_mn_major) return -12;         // not used by forward, dgrad or wgrad
  const int m_tiles = (M + 255) / 256;
  if (bn == 0) {
    // The 256-column tile moves a third fewer operand bytes per FLOP and measured faster on every training shape,
    // also where the 128-column tile has the fuller last wave; the narrow tile is for N <= 128.
    bn = N > 128 ? 256 : 128;
  }
  if (bn != 256 && bn != 128) return -13;
  G2Params p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc;
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.out_f32 = out_f32;
  p.status = status;
  int rc = a_mn_major ? tma_map_2d_bf16(&p.a_map, A, K, M, lda, G2_BK) : tma_map_2d_bf16(&p.a_map, A, M, K, lda, G2_BM);
  if (rc != 0) return -20 + rc;
  rc = b_mn_major ? tma_map_2d_bf16(&p.b_map, B, K, N, ldb, G2_BK) : tma_map_2d_bf16(&p.b_map, B, N, K, ldb, bn / 2);
  if (rc != 0) return -30 + rc;
  const int tiles = m_tiles * ((N + bn - 1) / bn);
  if (bn == 256) {
    if (!a_mn_major && !b_mn_major) return g2_launch<256, false, false>(p, tiles, stream);
    if (!a_mn_major && b_mn_major) return g2_launch<256, false, true>(p, tiles, stream);
    return g2_launch<256, true, true>(p, tiles, stream);
  }
  if (!a_mn_major && !b_mn_major) return g2_launch<128, false, false>(p, tiles, stream);
  if (!a_mn_major && b_mn_major) return g2_launch<128, false, true>(p, tiles, stream);
  return g2_launch<128, true, true>(p, tiles, stream);
}

// The same GEMM carrying the all-gather of a row-sharded matrix (see G2Params). consume != 0: B is ignored and the
// gathered matrix ([N, K], K-major, N / parts rows per part, which must be a multiple of 256) is the B operand;
// consume == 0: the launch computes its own product (the MN/MN weight gradient) and only carries the copy.
// gather_chunks: pieces a part is published in when consumed (1 = whole parts); the flag and counter arrays hold
// gather_parts * gather_chunks ints.
extern "C" int rb_gemm2_bf16_gather(const void* A, const void* B, void* C, const void* bias, const void* residual, int M, int N,
                                    int K, long long lda, long long ldb, long long ldc, long long ldr, int a_mn_major,
                                    int b_mn_major, int out_f32, const void* const* gather_src, void* gather_dst,
                                    long long gather_part_bytes, int* gather_count, int* gather_ready, int gather_epoch,
                                    int gather_parts, int rank, int consume, int gather_chunks, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || N % 8 != 0 || K % 8 != 0) return -1;
  if (gather_parts < 1 || gather_parts > 8 || rank < 0 || rank >= gather_parts || gather_dst == nullptr || gather_count == nullptr ||
      gather_ready == nullptr || gather_part_bytes <= 0 || gather_part_bytes % 16 != 0)
    return -1;
  if (a_mn_major != b_mn_major) return -12;                 // forward (K/K) and weight gradient (MN/MN) only
  if (consume && (a_mn_major || N % gather_parts != 0 || (N / gather_parts) % 256 != 0)) return -12;
  G2Params p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc;
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.out_f32 = out_f32;
  p.status = status;
  for (int r = 0; r < gather_parts; ++r) p.gather_src[r] = gather_src[r];
  p.gather_dst = gather_dst; p.gather_part_bytes = gather_part_bytes;
  p.gather_count = gather_count; p.gather_ready = gather_ready; p.gather_epoch = gather_epoch;
  p.gather_parts = gather_parts; p.rank = rank; p.consume = consume ? 1 : 0;
  p.n_tiles_per_part = consume ? (N / gather_parts) / 256 : 1;
  // gather_count / gather_ready hold gather_parts * gather_chunks entries (at most 64)
  if (!consume || gather_chunks < 1) gather_chunks = 1;
  if (gather_chunks > p.n_tiles_per_part) gather_chunks = p.n_tiles_per_part;
  while (gather_chunks > 1 && gather_parts * gather_chunks > 64) --gather_chunks;
  p.gather_chunk_tiles = consume ? (p.n_tiles_per_part + gather_chunks - 1) / gather_chunks : 1;
  p.gather_chunks = consume ? (p.n_tiles_per_part + p.gather_chunk_tiles - 1) / p.gather_chunk_tiles : 1;
  p.gather_chunk_bytes = consume ? (long long)p.gather_chunk_tiles * 256 * K * 2 : gather_part_bytes;
  if (consume && gather_part_bytes != (long long)(N / gather_parts) * K * 2) return -1;
  if (consume) { B = gather_dst; ldb = K; }
  int rc = a_mn_major ? tma_map_2d_bf16(&p.a_map, A, K, M, lda, G2_BK) : tma_map_2d_bf16(&p.a_map, A, M, K, lda, G2_BM);
  if (rc != 0) return -20 + rc;
  rc = b_mn_major ? tma_map_2d_bf16(&p.b_map, B, K, N, ldb, G2_BK) : tma_map_2d_bf16(&p.b_map, B, N, K, ldb, 128);
  if (rc != 0) return -30 + rc;
  const int tiles = ((M + 255) / 256) * ((N + 255) / 256);
  if (!a_mn_major) return g2_launch<256, false, false, true>(p, tiles, stream);
  return g2_launch<256, true, true, true>(p, tiles, stream);
}
