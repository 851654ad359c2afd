// Collectives written as kernels over peer (symmetric) memory on NVLink 5 / NVSwitch.
//
// Every rank maps every peer's communication buffers into its own address space; the kernels
// below move data with plain 16-byte peer loads / stores and synchronise with release/acquire
// flags at system scope. Every wait is bounded and reports through the status word.
//
//   symm_barrier        all ranks signal all peers and wait for all peers (epoch based)
//   symm_signal         one-way "my data is ready" flag to every peer
//   rs_reduce           gradient reduce-scatter: each rank PULLS its shard of every peer's bf16
//                       gradient bucket, sums in fp32, applies the 1/N scale, writes its fp32
//                       shard and per-CTA partial sums of squares (global grad norm), one pass
//   clip_coef           exchanges the per-rank sums of squares through peer memory and turns
//                       them into the clip coefficient, on the device (no host round trip)
//   adamw_allgather     sharded AdamW (fp32 master + moments) fused with the parameter
//                       all-gather: the updated bf16 values are PUSHED into every peer's full
//                       parameter buffer from inside the optimizer kernel
//   reshard_copy        trainer -> engine weight sync: one launch copies a table of 2-D
//                       segments from (peer) trainer shards into the engine's packed tensor-
//                       parallel layout (fused QKV / gate|up packing, row or column slices)
//
// Replaces: FSDP2 NCCL reduce-scatter + clip_grad_norm_ + torch AdamW + all-gather
// (rollouts/training/backends/fsdp.py:289-322, 398-452) and the per-tensor dist.broadcast /
// disk round trip of the weight sync (rollouts/training/weight_sync.py:233-282).
#include <climits>

#include "common.cuh"

#define RB_MAX_RANKS 8

namespace rb {

struct PeerPtrs { void* p[RB_MAX_RANKS]; };

// flags: each rank owns int flags[slots][world] in symmetric memory; peer r writes [slot][r].
// The epoch lives in device memory (counter) so that a barrier captured in a CUDA graph uses a
// fresh epoch on every replay: epoch = *counter + 1, stored back once every peer arrived.
__global__ void symm_barrier_kernel(PeerPtrs flags, int rank, int world, int slot, int epoch, int* counter,
                                    int* status, unsigned long long budget_ns) {
  __shared__ int ep;
  if (threadIdx.x == 0) ep = counter != nullptr ? *counter + 1 : epoch;
  __syncthreads();
  __threadfence_system();
  const int r = threadIdx.x;
  if (r < world) {
    st_release_sys(reinterpret_cast<int*>(flags.p[r]) + slot * world + rank, ep);
    wait_flag_ge(reinterpret_cast<const int*>(flags.p[rank]) + slot * world + r, ep, status, budget_ns);
  }
  __syncthreads();
  if (threadIdx.x == 0 && counter != nullptr) *counter = ep;
}
// Element-wise maximum of four integers over the ranks without leaving the device: every rank stores its values into
// every peer's exchange buffer (slot [epoch parity][source rank][4]), raises its flag there, waits (bounded) for all
// flags and reduces its own copy. out[0..3] = maxima, out[4] = 1 if every peer answered in time, else 0 (then the
// epoch is not advanced and nothing in the shared status word is touched: the caller decides what a silent peer means).
// Two parities suffice: a rank can start epoch e + 2 only after every peer has raised its flag of e + 1, which a peer
// does after reading the values of e.
__global__ void symm_agree_max_kernel(PeerPtrs xchg, PeerPtrs flags, int rank, int world, int slot, int* counter,
                                      int v0, int v1, int v2, int v3, int* out, unsigned long long budget_ns) {
  __shared__ int ep;
  __shared__ int ok_all;
  if (threadIdx.x == 0) { ep = *counter + 1; ok_all = 1; }
  __syncthreads();
  const int parity = ep & 1;
  const int r = threadIdx.x;
  if (r < world) {
    int* dst = reinterpret_cast<int*>(xchg.p[r]) + (parity * world + rank) * 4;
    st_relaxed_sys(dst + 0, v0); st_relaxed_sys(dst + 1, v1); st_relaxed_sys(dst + 2, v2); st_relaxed_sys(dst + 3, v3);
    __threadfence_system();
    st_release_sys(reinterpret_cast<int*>(flags.p[r]) + slot * world + rank, ep);
    if (!wait_flag_ge(reinterpret_cast<const int*>(flags.p[rank]) + slot * world + r, ep, nullptr, budget_ns)) ok_all = 0;   // no status word: out[4] reports
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int* mine = reinterpret_cast<const int*>(xchg.p[rank]) + parity * world * 4;
    int m[4] = {INT_MIN, INT_MIN, INT_MIN, INT_MIN};
    if (ok_all) {
      for (int q = 0; q < world; ++q)
        for (int i = 0; i < 4; ++i) m[i] = max(m[i], ld_relaxed_sys(mine + q * 4 + i));
      *counter = ep;
    }
    for (int i = 0; i < 4; ++i) out[i] = m[i];
    out[4] = ok_all;
  }
}
__global__ void symm_signal_kernel(PeerPtrs flags, int rank, int world, int slot, int epoch) {
  __threadfence_system();
  const int r = threadIdx.x;
  if (r < world) st_release_sys(reinterpret_cast<int*>(flags.p[r]) + slot * world + rank, epoch);
}
// Same signal with the epoch kept on the device (*counter + 1, stored back): a launch captured in a CUDA graph
// publishes a fresh epoch on every replay. Every rank replays the same launches, so the counters stay equal.
__global__ void symm_signal_counter_kernel(PeerPtrs flags, int rank, int world, int slot, int* counter) {
  __shared__ int ep;
  if (threadIdx.x == 0) ep = *counter + 1;
  __syncthreads();
  __threadfence_system();
  const int r = threadIdx.x;
  if (r < world) st_release_sys(reinterpret_cast<int*>(flags.p[r]) + slot * world + rank, ep);
  __syncthreads();
  if (threadIdx.x == 0) *counter = ep;
}
__global__ void symm_wait_kernel(const int* my_flags, int world, int slot, int epoch, int* status,
                                 unsigned long long budget_ns) {
  const int r = threadIdx.x;
  if (r < world) wait_flag_ge(my_flags + slot * world + r, epoch, status, budget_ns);
}

__device__ __forceinline__ uint4 ld_peer_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.relaxed.sys.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_peer_16(void* p, uint4 v) {
  asm volatile("st.global.relaxed.sys.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// ---- reduce-scatter of a bf16 gradient bucket into this rank's fp32 shard -----------------
// grads.p[r] : rank r's full bucket [n_total] bf16; this rank reduces [rank*n_shard, +n_shard)
// ready flags (slot) must be >= epoch for every peer before its bucket is read (my_flags == nullptr: the caller
// has already waited, e.g. with symm_wait on the same stream). shard_f32 == nullptr: only the sum of squares is
// wanted (one rank, whose AdamW reads the bf16 gradients directly). The peers' loads of one vector are all in
// flight before the first add.
// WT: the rank count when it is 1, 2, 4 or 8 (the loads of a vector then sit in exactly WT registers and the trip
// count per thread is chosen so that eight 16-byte loads are in flight), 0 = any rank count up to RB_MAX_RANKS.
// Register use decides this kernel: with the loads of 4 x 8 vectors held at once it needed 190 registers, one CTA
// per SM, and read at 0.9 TB/s; at 85 registers or fewer three CTAs per SM keep the memory system busy.
template <int WT>
__global__ void __launch_bounds__(256, 3)
rs_reduce_kernel(PeerPtrs grads, const int* my_flags, int slot, int epoch, int rank, int world, long long n_shard, float scale,
                 float* __restrict__ shard_f32, int accumulate, float* __restrict__ sumsq_partial, int* status,
                 unsigned long long budget_ns) {
  constexpr int WMAX = WT ? WT : RB_MAX_RANKS;
  constexpr int UNR = WT == 1 ? 4 : WT == 2 ? 2 : WT == 4 ? 2 : 1;
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  if (my_flags != nullptr && threadIdx.x < world) {
    if (!wait_flag_ge(my_flags + slot * world + threadIdx.x, epoch, status, budget_ns)) failed = 1;
  }
  __syncthreads();
  float acc_sq = 0.f;
  if (!failed) {
    const long long nvec = n_shard >> 3;
    const long long base = (long long)rank * n_shard;
    const long long stride = (long long)gridDim.x * blockDim.x;
    // source pointers of this rank's slice, own bucket first, then the peers in ring order (links are used evenly)
    const __nv_bfloat16* src[WMAX];
#pragma unroll
    for (int rr = 0; rr < WMAX; ++rr) {
      int q = rank + rr;
      if (q >= world) q -= world;
      src[rr] = reinterpret_cast<const __nv_bfloat16*>(grads.p[rr < world ? q : rank]) + base;
    }
    for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < nvec; i0 += stride * UNR) {
      uint4 part[UNR][WMAX];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const long long i = i0 + u * stride;
        if (i < nvec) {
#pragma unroll
          for (int rr = 0; rr < WMAX; ++rr) {
            if (rr < world) {
              // this rank's own bucket was written by kernels earlier on this GPU: an ordinary streaming load; a
              // peer's bucket is read at system scope
              part[u][rr] = rr == 0 ? __ldcs(reinterpret_cast<const uint4*>(src[0] + i * 8)) : ld_peer_16(src[rr] + i * 8);
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const long long i = i0 + u * stride;
        if (i >= nvec) break;
        float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int rr = 0; rr < WMAX; ++rr) {
          if (rr < world) {
            const uint4 v = part[u][rr];
            float2 f;
            f = unpack_bf16x2(v.x); s[0] += f.x; s[1] += f.y;
            f = unpack_bf16x2(v.y); s[2] += f.x; s[3] += f.y;
            f = unpack_bf16x2(v.z); s[4] += f.x; s[5] += f.y;
            f = unpack_bf16x2(v.w); s[6] += f.x; s[7] += f.y;
          }
        }
        float4 a = make_float4(s[0] * scale, s[1] * scale, s[2] * scale, s[3] * scale);
        float4 b = make_float4(s[4] * scale, s[5] * scale, s[6] * scale, s[7] * scale);
        if (shard_f32 != nullptr) {
          float* o = shard_f32 + i * 8;
          if (accumulate) {
            const float4 pa = *reinterpret_cast<float4*>(o), pb = *reinterpret_cast<float4*>(o + 4);
            a.x += pa.x; a.y += pa.y; a.z += pa.z; a.w += pa.w;
            b.x += pb.x; b.y += pb.y; b.z += pb.z; b.w += pb.w;
          }
          *reinterpret_cast<float4*>(o) = a;
          *reinterpret_cast<float4*>(o + 4) = b;
        }
        acc_sq += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w + b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
      }
    }
  }
  // block reduce of the squares
  __shared__ float sm[32];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  acc_sq = warp_sum(acc_sq);
  if (lane == 0) sm[wid] = acc_sq;
  __syncthreads();
  if (wid == 0) {
    float r = lane < (blockDim.x >> 5) ? sm[lane] : 0.f;
    r = warp_sum(r);
    if (lane == 0 && sumsq_partial != nullptr) sumsq_partial[blockIdx.x] += r;
  }
}

// ---- global grad norm -> clip coefficient, exchanged through peer memory ---------------------
// partial: [n_partial] this rank's sums of squares. norm_slots.p[r]: rank r's float slots[world].
// out_coef = pre_scale * min(1, max_norm / (pre_scale * norm + 1e-6)): what AdamW multiplies the stored gradients by.
__global__ void clip_coef_kernel(const float* __restrict__ partial, int n_partial, PeerPtrs norm_slots, PeerPtrs flags,
                                 int slot, int epoch, int rank, int world, float max_norm, float pre_scale,
                                 float* __restrict__ out_coef, float* __restrict__ out_norm, int* status,
                                 unsigned long long budget_ns) {
  __shared__ float sm[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < n_partial; i += blockDim.x) acc += partial[i];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  acc = warp_sum(acc);
  if (lane == 0) sm[wid] = acc;
  __syncthreads();
  if (wid == 0) {
    float r = lane < (blockDim.x >> 5) ? sm[lane] : 0.f;
    r = warp_sum(r);
    if (lane == 0) sm[0] = r;
  }
  __syncthreads();
  const float mine = sm[0];
  const int r = threadIdx.x;
  if (r < world) {
    reinterpret_cast<float*>(norm_slots.p[r])[rank] = mine;
    __threadfence_system();
    st_release_sys(reinterpret_cast<int*>(flags.p[r]) + slot * world + rank, epoch);
  }
  __syncthreads();
  bool ok = true;
  if (r < world) ok = wait_flag_ge(reinterpret_cast<const int*>(flags.p[rank]) + slot * world + r, epoch, status, budget_ns);
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.f;
    const volatile float* slots = reinterpret_cast<const volatile float*>(norm_slots.p[rank]);
    for (int i = 0; i < world; ++i) total += slots[i];
    // pre_scale: the sums were taken over gradients that still carry a common factor (1 / accumulated passes);
    // the norm is reported for the scaled gradients and the factor rides in the coefficient
    const float norm = sqrtf(total) * pre_scale;
    *out_norm = norm;
    *out_coef = pre_scale * ((max_norm > 0.f) ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f);
  }
  (void)ok;
}

// ---- sharded AdamW fused with the parameter all-gather ------------------------------------------
// params.p[r]: rank r's full bf16 parameter bucket [n_total]; this rank owns [rank*n_shard, +n_shard).
// VEC: the four fp32 streams are read and written as float4 (needs 16-byte aligned base pointers); otherwise each
// thread walks its eight elements with scalar accesses.
// GBF16: `grad` is this rank's slice of the bf16 gradient bucket itself (one rank: nothing was reduced, so no fp32
// copy of the gradients exists); the common scale rides in *clip_coef.
template <bool VEC, bool GBF16>
__global__ void adamw_allgather_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                                       const void* __restrict__ grad_any, PeerPtrs params, int rank, int world,
                                       long long n_shard, float lr, float beta1, float beta2, float eps,
                                       float weight_decay, float bc1, float bc2, const float* __restrict__ clip_coef) {
  const float clip = clip_coef != nullptr ? *clip_coef : 1.f;
  const long long nvec = n_shard >> 3;
  const long long base = (long long)rank * n_shard;
  const float decay = 1.f - lr * weight_decay, ibc1 = 1.f / bc1, ibc2 = 1.f / bc2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float g8[8], m8[8], v8[8], p8[8];
    const float* grad = reinterpret_cast<const float*>(grad_any);
    if constexpr (GBF16) {
      const uint4 gv = *(reinterpret_cast<const uint4*>(grad_any) + i);
      float2 f;
      f = unpack_bf16x2(gv.x); g8[0] = f.x; g8[1] = f.y;
      f = unpack_bf16x2(gv.y); g8[2] = f.x; g8[3] = f.y;
      f = unpack_bf16x2(gv.z); g8[4] = f.x; g8[5] = f.y;
      f = unpack_bf16x2(gv.w); g8[6] = f.x; g8[7] = f.y;
    }
    if constexpr (VEC) {
      const float4* g4 = reinterpret_cast<const float4*>(grad) + 2 * i;
      const float4* m4 = reinterpret_cast<const float4*>(m) + 2 * i;
      const float4* v4 = reinterpret_cast<const float4*>(v) + 2 * i;
      const float4* p4 = reinterpret_cast<const float4*>(master) + 2 * i;
      if constexpr (!GBF16) {
        *reinterpret_cast<float4*>(g8) = g4[0];
        *reinterpret_cast<float4*>(g8 + 4) = g4[1];
      }
      *reinterpret_cast<float4*>(m8) = m4[0];
      *reinterpret_cast<float4*>(m8 + 4) = m4[1];
      *reinterpret_cast<float4*>(v8) = v4[0];
      *reinterpret_cast<float4*>(v8 + 4) = v4[1];
      *reinterpret_cast<float4*>(p8) = p4[0];
      *reinterpret_cast<float4*>(p8 + 4) = p4[1];
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const long long k = i * 8 + j;
        if constexpr (!GBF16) g8[j] = grad[k];
        m8[j] = m[k];
        v8[j] = v[k];
        p8[j] = master[k];
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float g = g8[j] * clip;
      m8[j] = beta1 * m8[j] + (1.f - beta1) * g;
      v8[j] = beta2 * v8[j] + (1.f - beta2) * g * g;
      p8[j] = p8[j] * decay - lr * (m8[j] * ibc1) / (sqrtf(v8[j] * ibc2) + eps);
    }
    if constexpr (VEC) {
      float4* m4 = reinterpret_cast<float4*>(m) + 2 * i;
      float4* v4 = reinterpret_cast<float4*>(v) + 2 * i;
      float4* p4 = reinterpret_cast<float4*>(master) + 2 * i;
      m4[0] = *reinterpret_cast<float4*>(m8);
      m4[1] = *reinterpret_cast<float4*>(m8 + 4);
      v4[0] = *reinterpret_cast<float4*>(v8);
      v4[1] = *reinterpret_cast<float4*>(v8 + 4);
      p4[0] = *reinterpret_cast<float4*>(p8);
      p4[1] = *reinterpret_cast<float4*>(p8 + 4);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const long long k = i * 8 + j;
        m[k] = m8[j];
        v[k] = v8[j];
        master[k] = p8[j];
      }
    }
    uint4 o;
    o.x = pack_bf16x2(p8[0], p8[1]);
    o.y = pack_bf16x2(p8[2], p8[3]);
    o.z = pack_bf16x2(p8[4], p8[5]);
    o.w = pack_bf16x2(p8[6], p8[7]);
    for (int rr = 0; rr < world; ++rr) {
      const int dst = (rank + rr) % world;
      st_peer_16(reinterpret_cast<__nv_bfloat16*>(params.p[dst]) + base + i * 8, o);
    }
  }
}

// ---- weight reshard copy ---------------------------------------------------------------------------
struct Segment {
  const void* src;     // bf16, may be peer memory
  void* dst;           // bf16, local
  long long src_ld, dst_ld;   // elements
  int rows, cols;      // cols multiple of 8
  long long vec_begin; // prefix sum of rows * cols / 8
};

__global__ void reshard_copy_kernel(const Segment* __restrict__ segs, int n_segs, long long total_vecs) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total_vecs;
       i += (long long)gridDim.x * blockDim.x) {
    int lo = 0, hi = n_segs - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (segs[mid].vec_begin <= i) lo = mid; else hi = mid - 1;
    }
    const Segment s = segs[lo];
    const long long k = i - s.vec_begin;
    const int vpr = s.cols >> 3;
    const long long r = k / vpr;
    const int c = (int)(k % vpr) * 8;
    const uint4 v = ld_peer_16(reinterpret_cast<const __nv_bfloat16*>(s.src) + r * s.src_ld + c);
    *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(s.dst) + r * s.dst_ld + c) = v;
  }
}

}  // namespace rb

using namespace rb;
#define RB_OK() (cudaGetLastError() == cudaSuccess ? 0 : -11)

static PeerPtrs make_ptrs(void* const* p, int world) {
  PeerPtrs o;
  for (int i = 0; i < RB_MAX_RANKS; ++i) o.p[i] = i < world ? p[i] : nullptr;
  return o;
}

namespace rb {
// Pull-based sum of one bf16 tile held by every rank: out = residual + sum_r src[r], fp32 accumulation in rank order
// (the same order on every rank, so all ranks end with identical bits). src[r] are peer mappings of the ranks' slabs;
// the caller's device barrier has made them complete. 16-byte vectors.
__global__ void pull_sum_kernel(PeerPtrs src, const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ out,
                                long long nvec, int world) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float acc[8];
    {
      const uint4 r = reinterpret_cast<const uint4*>(residual)[i];
      const uint32_t ri[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(ri[j]);
        acc[2 * j] = f.x; acc[2 * j + 1] = f.y;
      }
    }
    uint4 part[RB_MAX_RANKS];
#pragma unroll
    for (int r = 0; r < RB_MAX_RANKS; ++r)
      if (r < world) part[r] = reinterpret_cast<const uint4*>(src.p[r])[i];     // all loads in flight before the adds
#pragma unroll
    for (int r = 0; r < RB_MAX_RANKS; ++r) {
      if (r < world) {
        const uint32_t pi[4] = {part[r].x, part[r].y, part[r].z, part[r].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(pi[j]);
          acc[2 * j] += f.x; acc[2 * j + 1] += f.y;
        }
      }
    }
    reinterpret_cast<uint4*>(out)[i] = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                                                  pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
  }
}

// The same sum with its synchronisation inside the launch (tensor-parallel all-reduce of decode-sized outputs as
// GEMM + this kernel, nothing else): block 0 tells every peer that this rank's slab is complete (the GEMM before this
// launch on the stream wrote it), every block waits (bounded) for all peers' flags, sums, and the last block to
// finish tells every peer that their slabs have been read (one increment of the peer's acknowledgement counter per
// call) and raises the count this rank's NEXT slab write has to wait for (`need`, consumed by the GEMM's producer).
// Epochs and tickets live on the device, so a captured launch replays correctly. sync: [0] epoch, [1] ticket.
__global__ void pull_sum_sync_kernel(PeerPtrs src, const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ out,
                                     long long nvec, int world, int rank, PeerPtrs flags, int slot, int* sync, PeerPtrs ack,
                                     int* need, int* status, unsigned long long budget_ns) {
  __shared__ int ep_s;
  __shared__ int failed;
  if (threadIdx.x == 0) { ep_s = ld_relaxed_sys(sync) + 1; failed = 0; }
  __syncthreads();
  const int ep = ep_s;
  if (blockIdx.x == 0 && threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<int*>(flags.p[threadIdx.x]) + slot * world + rank, ep);
  }
  if (threadIdx.x < world && threadIdx.x != rank) {
    if (!wait_flag_ge(reinterpret_cast<const int*>(flags.p[rank]) + slot * world + threadIdx.x, ep, status, budget_ns)) failed = 1;
  }
  __syncthreads();
  if (!failed) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
      float acc[8];
      {
        const uint4 r = reinterpret_cast<const uint4*>(residual)[i];
        const uint32_t ri[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(ri[j]);
          acc[2 * j] = f.x; acc[2 * j + 1] = f.y;
        }
      }
      uint4 part[RB_MAX_RANKS];
#pragma unroll
      for (int r = 0; r < RB_MAX_RANKS; ++r)
        if (r < world) part[r] = ld_peer_16(reinterpret_cast<const uint4*>(src.p[r]) + i);   // rank order: same bits on every rank
#pragma unroll
      for (int r = 0; r < RB_MAX_RANKS; ++r) {
        if (r < world) {
          const uint32_t pi[4] = {part[r].x, part[r].y, part[r].z, part[r].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = unpack_bf16x2(pi[j]);
            acc[2 * j] += f.x; acc[2 * j + 1] += f.y;
          }
        }
      }
      reinterpret_cast<uint4*>(out)[i] = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                                                    pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int old = atomicAdd(sync + 1, 1);
    if (old == (int)gridDim.x - 1) {          // every block of this launch is done reading the peers' slabs
      sync[1] = 0;
      if (!failed) {
        sync[0] = ep;
        *need += world - 1;
        __threadfence_system();
        for (int r = 0; r < world; ++r)
          if (r != rank) asm volatile("red.release.sys.global.add.s32 [%0], 1;" ::"l"(reinterpret_cast<int*>(ack.p[r])) : "memory");
      }
    }
  }
}
}  // namespace rb
using namespace rb;

extern "C" int rb_pull_sum(void* const* src_ptrs, const void* residual, void* out, long long n, int world, cudaStream_t s) {
  if (world < 1 || world > RB_MAX_RANKS || n <= 0 || n % 8 != 0) return -1;
  const long long nvec = n / 8;
  long long grid = (nvec + 255) / 256;
  if (grid > 148 * 4) grid = 148 * 4;
  pull_sum_kernel<<<(unsigned)grid, 256, 0, s>>>(make_ptrs(src_ptrs, world), (const __nv_bfloat16*)residual, (__nv_bfloat16*)out,
                                                 nvec, world);
  return RB_OK();
}

static unsigned long long g_wait_budget_ns = RB_WAIT_BUDGET_NS;
// Budget of every cross-GPU flag wait launched through this library from now on (nanoseconds; 0 restores the
// default). A wait that runs out records ST_TIMEOUT_PEER_FLAG in the status word and the kernel returns.
extern "C" void rb_comm_set_wait_budget_ns(unsigned long long ns) { g_wait_budget_ns = ns ? ns : RB_WAIT_BUDGET_NS; }
extern "C" unsigned long long rb_comm_get_wait_budget_ns() { return g_wait_budget_ns; }

extern "C" int rb_symm_barrier(void* const* flag_ptrs, int rank, int world, int slot, int epoch, int* counter,
                               int* status, cudaStream_t s) {
  if (world < 1 || world > RB_MAX_RANKS) return -1;
  symm_barrier_kernel<<<1, 32, 0, s>>>(make_ptrs(flag_ptrs, world), rank, world, slot, epoch, counter, status, g_wait_budget_ns);
  return RB_OK();
}
extern "C" int rb_pull_sum_sync(void* const* src_ptrs, const void* residual, void* out, long long n, int world, int rank,
                                void* const* flag_ptrs, int slot, int* sync, void* const* ack_ptrs, int* need, int* status,
                                cudaStream_t s) {
  if (world < 1 || world > RB_MAX_RANKS || n <= 0 || n % 8 != 0 || sync == nullptr || need == nullptr) return -1;
  const long long nvec = n / 8;
  long long grid = (nvec + 255) / 256;
  if (grid > 148 * 2) grid = 148 * 2;      // every block must be resident: they all wait for the peers
  pull_sum_sync_kernel<<<(unsigned)grid, 256, 0, s>>>(make_ptrs(src_ptrs, world), (const __nv_bfloat16*)residual, (__nv_bfloat16*)out,
                                                      nvec, world, rank, make_ptrs(flag_ptrs, world), slot, sync,
                                                      make_ptrs(ack_ptrs, world), need, status, g_wait_budget_ns);
  return RB_OK();
}
extern "C" int rb_symm_agree_max(void* const* xchg_ptrs, void* const* flag_ptrs, int rank, int world, int slot, int* counter,
                                 int v0, int v1, int v2, int v3, int* out, unsigned long long budget_ns, cudaStream_t s) {
  if (world < 1 || world > RB_MAX_RANKS || counter == nullptr || out == nullptr) return -1;
  symm_agree_max_kernel<<<1, 32, 0, s>>>(make_ptrs(xchg_ptrs, world), make_ptrs(flag_ptrs, world), rank, world, slot, counter,
                                         v0, v1, v2, v3, out, budget_ns ? budget_ns : g_wait_budget_ns);
  return RB_OK();
}
extern "C" int rb_symm_signal(void* const* flag_ptrs, int rank, int world, int slot, int epoch, cudaStream_t s) {
  if (world < 1 || world > RB_MAX_RANKS) return -1;
  symm_signal_kernel<<<1, 32, 0, s>>>(make_ptrs(flag_ptrs, world), rank, world, slot, epoch);
  return RB_OK();
}
extern "C" int rb_symm_signal_counter(void* const* flag_ptrs, int rank, int world, int slot, int* counter, cudaStream_t s) {
  if (world < 1 || world > RB_MAX_RANKS || counter == nullptr) return -1;
  symm_signal_counter_kernel<<<1, 32, 0, s>>>(make_ptrs(flag_ptrs, world), rank, world, slot, counter);
  return RB_OK();
}
extern "C" int rb_symm_wait(const int* my_flags, int world, int slot, int epoch, int* status, cudaStream_t s) {
  symm_wait_kernel<<<1, 32, 0, s>>>(my_flags, world, slot, epoch, status, g_wait_budget_ns);
  return RB_OK();
}
// Same wait with its own budget (the failure branch of the bounded wait is tested with a millisecond).
extern "C" int rb_symm_wait_budget(const int* my_flags, int world, int slot, int epoch, int* status,
                                   unsigned long long budget_ns, cudaStream_t s) {
  if (world < 1 || world > 32) return -1;
  symm_wait_kernel<<<1, 32, 0, s>>>(my_flags, world, slot, epoch, status, budget_ns);
  return RB_OK();
}
extern "C" int rb_rs_num_partials() { return 148 * 4; }
// grid_ctas: 0 = one CTA per partial slot (a launch that has the GPU to itself); a launch that shares the SMs with
// the backward pass asks for fewer. my_flags may be null when the caller has waited already; shard_f32 may be null
// when only the sum of squares is wanted.
extern "C" int rb_rs_reduce_ex(void* const* grad_ptrs, const int* my_flags, int slot, int epoch, int rank, int world,
                               long long n_shard, float scale, float* shard_f32, int accumulate, float* sumsq_partial,
                               int* status, int grid_ctas, cudaStream_t s) {
  if (world < 1 || world > RB_MAX_RANKS || n_shard % 8 != 0) return -1;
  if (shard_f32 == nullptr && accumulate) return -1;
  int grid = grid_ctas > 0 ? grid_ctas : rb_rs_num_partials();
  if (grid > rb_rs_num_partials()) grid = rb_rs_num_partials();
  const PeerPtrs pp = make_ptrs(grad_ptrs, world);
#define RB_RS_LAUNCH(WT) rs_reduce_kernel<WT><<<grid, 256, 0, s>>>(pp, my_flags, slot, epoch, rank, world, n_shard, scale, shard_f32, \
                                                                  accumulate, sumsq_partial, status, g_wait_budget_ns)
  switch (world) {
    case 1: RB_RS_LAUNCH(1); break;
    case 2: RB_RS_LAUNCH(2); break;
    case 4: RB_RS_LAUNCH(4); break;
    case 8: RB_RS_LAUNCH(8); break;
    default: RB_RS_LAUNCH(0); break;
  }
#undef RB_RS_LAUNCH
  return RB_OK();
}
extern "C" int rb_rs_reduce(void* const* grad_ptrs, const int* my_flags, int slot, int epoch, int rank, int world,
                            long long n_shard, float scale, float* shard_f32, int accumulate, float* sumsq_partial,
                            int* status, cudaStream_t s) {
  return rb_rs_reduce_ex(grad_ptrs, my_flags, slot, epoch, rank, world, n_shard, scale, shard_f32, accumulate, sumsq_partial,
                         status, 0, s);
}
extern "C" int rb_clip_coef_ex(const float* partial, int n_partial, void* const* norm_slot_ptrs, void* const* flag_ptrs,
                               int slot, int epoch, int rank, int world, float max_norm, float pre_scale, float* out_coef,
                               float* out_norm, int* status, cudaStream_t s) {
  if (world < 1 || world > RB_MAX_RANKS) return -1;
  clip_coef_kernel<<<1, 256, 0, s>>>(partial, n_partial, make_ptrs(norm_slot_ptrs, world), make_ptrs(flag_ptrs, world),
                                     slot, epoch, rank, world, max_norm, pre_scale, out_coef, out_norm, status, g_wait_budget_ns);
  return RB_OK();
}
extern "C" int rb_clip_coef(const float* partial, int n_partial, void* const* norm_slot_ptrs, void* const* flag_ptrs,
                            int slot, int epoch, int rank, int world, float max_norm, float* out_coef, float* out_norm,
                            int* status, cudaStream_t s) {
  return rb_clip_coef_ex(partial, n_partial, norm_slot_ptrs, flag_ptrs, slot, epoch, rank, world, max_norm, 1.f, out_coef,
                         out_norm, status, s);
}
// grad_is_bf16: `grad` points at this rank's slice of the bf16 gradient bucket instead of an fp32 reduced copy.
extern "C" int rb_adamw_allgather_ex(float* master, float* m, float* v, const void* grad, int grad_is_bf16,
                                     void* const* param_ptrs, int rank, int world, long long n_shard, float lr, float beta1,
                                     float beta2, float eps, float weight_decay, int step, const float* clip_coef,
                                     cudaStream_t s) {
  if (world < 1 || world > RB_MAX_RANKS || n_shard % 8 != 0) return -1;
  if (n_shard == 0) return 0;
  const float bc1 = 1.f - powf(beta1, (float)step), bc2 = 1.f - powf(beta2, (float)step);
  const bool aligned = ((reinterpret_cast<uintptr_t>(master) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
                         reinterpret_cast<uintptr_t>(grad)) & 15) == 0;
  const PeerPtrs pp = make_ptrs(param_ptrs, world);
  if (grad_is_bf16) {
    if (!aligned) return -2;
    adamw_allgather_kernel<true, true><<<148 * 8, 256, 0, s>>>(master, m, v, grad, pp, rank, world, n_shard, lr, beta1, beta2,
                                                               eps, weight_decay, bc1, bc2, clip_coef);
  } else if (aligned) {
    adamw_allgather_kernel<true, false><<<148 * 8, 256, 0, s>>>(master, m, v, grad, pp, rank, world, n_shard, lr, beta1, beta2,
                                                                eps, weight_decay, bc1, bc2, clip_coef);
  } else {
    adamw_allgather_kernel<false, false><<<148 * 4, 256, 0, s>>>(master, m, v, grad, pp, rank, world, n_shard, lr, beta1, beta2,
                                                                 eps, weight_decay, bc1, bc2, clip_coef);
  }
  return RB_OK();
}
extern "C" int rb_adamw_allgather(float* master, float* m, float* v, const float* grad, void* const* param_ptrs,
                                  int rank, int world, long long n_shard, float lr, float beta1, float beta2, float eps,
                                  float weight_decay, int step, const float* clip_coef, cudaStream_t s) {
  return rb_adamw_allgather_ex(master, m, v, grad, 0, param_ptrs, rank, world, n_shard, lr, beta1, beta2, eps, weight_decay,
                               step, clip_coef, s);
}
// segs: device array of Segment (layout mirrored by research_b200/parallel/weight_sync.py)
extern "C" int rb_reshard_copy(const void* segs, int n_segs, long long total_vecs, cudaStream_t s) {
  if (n_segs <= 0 || total_vecs <= 0) return 0;
  long long grid = (total_vecs + 255) / 256;
  if (grid > 148 * 8) grid = 148 * 8;
  reshard_copy_kernel<<<(unsigned)grid, 256, 0, s>>>((const Segment*)segs, n_segs, total_vecs);
  return RB_OK();
}
