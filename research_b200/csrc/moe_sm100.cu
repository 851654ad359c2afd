// Mixture-of-experts routing and token movement for sm_100a.
//
//   moe_route      softmax-top-k (Qwen3-MoE: softmax over all experts, top-k, renormalise) or
//                  sigmoid + correction-bias top-k (GLM-4-MoE), one warp per token
//   moe_plan       per-expert counts -> offsets, and the tile table of the grouped GEMM
//                  (entries {a_row0, valid_rows, b_row0, n0}) built on the device so the
//                  whole layer stays inside one CUDA graph
//   moe_permute    scatter token rows into expert-contiguous order; the destination may be the
//                  receive buffer of the expert's owner GPU (dispatch over peer memory), and
//                  each row records where its result has to be written back
//   moe_combine    out[t] += sum_j w[t,j] * y[t*k + j]
//
// The expert GEMMs themselves are the grouped mode of csrc/gemm_sm100.cu; with row_dst set, the
// down-projection epilogue stores every result row straight into the token's home buffer
// (local or on the source GPU), which is the combine half of the all-to-all.
//
// Math oracles: rollouts/tools/functional_extractor/qwen3_next_functional.py:409-490 (softmax
// top-k) and glm4_moe_functional.py:230-369 (sigmoid router, per-expert loop with index_add_).
#include "common.cuh"

#define RB_MAX_RANKS 8

namespace rb {

constexpr int MAX_E_PER_LANE = 8;  // up to 256 experts

// n_group > 1 (sigmoid router only): group-limited routing. Experts form n_group contiguous groups, a group scores
// the sum of its two best choice values, the topk_group best groups stay eligible and the choice values of the
// other experts become 0 (glm4_moe_functional.py:278-301).
__global__ void moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int T, int E,
                                 int k, int sigmoid_router, int norm_topk, float scaling, int* __restrict__ topk_idx,
                                 float* __restrict__ topk_w, int* __restrict__ counts /*[E] histogram, may be null*/,
                                 int n_group, int topk_group) {
  __shared__ int hist[256];
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (counts != nullptr) {
    for (int i = threadIdx.x; i < E; i += blockDim.x) hist[i] = 0;
    __syncthreads();
  }
  if (t < T) {
  float score[MAX_E_PER_LANE], choice[MAX_E_PER_LANE];
  const int per = (E + 31) / 32;
  float mx = -INFINITY;
  for (int i = 0; i < per; ++i) {
    const int e = lane + 32 * i;
    const float x = e < E ? logits[(long long)t * E + e] : -INFINITY;
    score[i] = x;
    mx = fmaxf(mx, x);
  }
  if (sigmoid_router) {
    for (int i = 0; i < per; ++i) {
      const int e = lane + 32 * i;
      score[i] = e < E ? 1.f / (1.f + __expf(-score[i])) : -INFINITY;
      choice[i] = e < E ? score[i] + (bias != nullptr ? bias[e] : 0.f) : -INFINITY;
    }
    if (n_group > 1 && topk_group < n_group) {
      const int gsz = E / n_group;
      float my_g = -INFINITY;                       // lane g keeps the score of group g (n_group <= 32)
      for (int g = 0; g < n_group; ++g) {
        float m1 = -INFINITY, m2 = -INFINITY;       // the two best choice values of this lane's experts in group g
        for (int i = 0; i < per; ++i) {
          const int e = lane + 32 * i;
          if (e < E && e / gsz == g) {
            const float c = choice[i];
            if (c > m1) { m2 = m1; m1 = c; } else if (c > m2) { m2 = c; }
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {          // merge top-2 pairs of disjoint lane sets
          const float a1 = __shfl_xor_sync(0xffffffffu, m1, o);
          const float a2 = __shfl_xor_sync(0xffffffffu, m2, o);
          m2 = fmaxf(fminf(m1, a1), fmaxf(m2, a2));
          m1 = fmaxf(m1, a1);
        }
        if (lane == g) my_g = m1 + m2;
      }
      unsigned keep = 0u;
      for (int j = 0; j < topk_group; ++j) {
        float best = my_g;
        int best_g = lane;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float b2 = __shfl_xor_sync(0xffffffffu, best, o);
          const int g2 = __shfl_xor_sync(0xffffffffu, best_g, o);
          if (b2 > best || (b2 == best && g2 < best_g)) { best = b2; best_g = g2; }
        }
        keep |= 1u << best_g;
        if (lane == best_g) my_g = -INFINITY;
      }
      for (int i = 0; i < per; ++i) {
        const int e = lane + 32 * i;
        if (e < E && !((keep >> (e / gsz)) & 1u)) choice[i] = 0.f;
      }
    }
  } else {
    mx = warp_max(mx);
    float sum = 0.f;
    for (int i = 0; i < per; ++i) {
      const int e = lane + 32 * i;
      score[i] = e < E ? __expf(score[i] - mx) : 0.f;
      sum += score[i];
    }
    sum = warp_sum(sum);
    for (int i = 0; i < per; ++i) {
      score[i] /= sum;
      choice[i] = (lane + 32 * i) < E ? score[i] : -INFINITY;
    }
  }
  float wsum = 0.f;
  float my_w = 0.f;
  int my_e = 0;
  for (int j = 0; j < k; ++j) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int i = 0; i < per; ++i) {
      const int e = lane + 32 * i;
      if (choice[i] > best || (choice[i] == best && e < best_e)) { best = choice[i]; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float b2 = __shfl_xor_sync(0xffffffffu, best, o);
      const int e2 = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (b2 > best || (b2 == best && e2 < best_e)) { best = b2; best_e = e2; }
    }
    // the owner lane reports the (un-biased) score and retires the expert
    float w = 0.f;
    if ((best_e & 31) == lane) {
      const int i = best_e >> 5;
      w = score[i];
      choice[i] = -INFINITY;
    }
    w = __shfl_sync(0xffffffffu, w, best_e & 31);
    wsum += w;
    if (lane == j) { my_w = w; my_e = best_e; }
  }
  if (lane < k) {
    float w = my_w;
    if (norm_topk) w = w / (wsum + 1e-20f);
    topk_idx[(long long)t * k + lane] = my_e;
    topk_w[(long long)t * k + lane] = w * scaling;
    if (counts != nullptr) atomicAdd(&hist[my_e], 1);
  }
  }
  if (counts != nullptr) {   // integer adds: the histogram does not depend on their order
    __syncthreads();
    for (int i = threadIdx.x; i < E; i += blockDim.x)
      if (hist[i]) atomicAdd(&counts[i], hist[i]);
  }
}

// counts_all: [world][E] rows routed from each source rank to each expert (world = 1 locally).
// Experts [e_lo, e_hi) are owned by this rank. Outputs (for the owned experts): offsets of each
// expert's row block in the local expert-ordered buffer and the grouped-GEMM tile tables for
// two GEMMs with different N (gate|up and down), all built by one CTA.
__global__ void moe_plan_kernel(const int* __restrict__ counts_all, int world, int E, int e_lo, int e_hi,
                                int* __restrict__ expert_offset /*[E_local+1]*/, int n_gu, int bn_gu,
                                int4* __restrict__ tiles_gu, int* __restrict__ ntiles_gu, int n_dn, int bn_dn,
                                int4* __restrict__ tiles_dn, int* __restrict__ ntiles_dn, int max_tiles,
                                int* status, int rank, int* __restrict__ cursor /*[2E] or null: [E..2E) = send bases*/) {
  __shared__ int cnt[256], off[257], tb_gu[257], tb_dn[257];
  const int EL = e_hi - e_lo;
  if (cursor != nullptr) {
    // where this rank's rows for expert e start in the owner's expert-ordered receive buffer: the rows of the
    // owner's lower experts (from all ranks) plus the rows of lower source ranks for e. Column sums go through
    // shared memory first so that no thread walks the count matrix serially.
    __shared__ int tot[256], below[256];
    const int epr = E / world;
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
      int a = 0, b = 0;
      for (int r = 0; r < world; ++r) {
        const int c = counts_all[r * E + e];
        a += c;
        if (r < rank) b += c;
      }
      tot[e] = a; below[e] = b;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
      int o = below[e];
      for (int ee = (e / epr) * epr; ee < e; ++ee) o += tot[ee];
      cursor[E + e] = o;
    }
  }
  for (int i = threadIdx.x; i < EL; i += blockDim.x) {
    int c = 0;
    for (int r = 0; r < world; ++r) c += counts_all[r * E + e_lo + i];
    cnt[i] = c;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int o = 0, tg = 0, td = 0;
    const int ngu = (n_gu + bn_gu - 1) / bn_gu, ndn = (n_dn + bn_dn - 1) / bn_dn;
    for (int i = 0; i < EL; ++i) {
      off[i] = o; tb_gu[i] = tg; tb_dn[i] = td;
      const int mt = (cnt[i] + 127) / 128;
      o += cnt[i]; tg += mt * ngu; td += mt * ndn;
    }
    off[EL] = o; tb_gu[EL] = tg; tb_dn[EL] = td;
    if (tg > max_tiles || td > max_tiles) { set_status(status, ST_BAD_INDEX); tg = min(tg, max_tiles); td = min(td, max_tiles); }
    *ntiles_gu = tg; *ntiles_dn = td;
  }
  __syncthreads();
  for (int i = threadIdx.x; i <= EL; i += blockDim.x) expert_offset[i] = off[i];
  const int ngu = (n_gu + bn_gu - 1) / bn_gu, ndn = (n_dn + bn_dn - 1) / bn_dn;
  for (int i = threadIdx.x; i < EL; i += blockDim.x) {
    const int mt = (cnt[i] + 127) / 128;
    for (int m = 0; m < mt; ++m) {
      const int rows = min(128, cnt[i] - m * 128);
      for (int n = 0; n < ngu; ++n) {
        const int idx = tb_gu[i] + m * ngu + n;
        if (idx < max_tiles) tiles_gu[idx] = make_int4(off[i] + m * 128, rows, i * n_gu + n * bn_gu, n * bn_gu);
      }
      for (int n = 0; n < ndn; ++n) {
        const int idx = tb_dn[i] + m * ndn + n;
        if (idx < max_tiles) tiles_dn[idx] = make_int4(off[i] + m * 128, rows, i * n_dn + n * bn_dn, n * bn_dn);
      }
    }
  }
}

// Per-expert histogram of this rank's routing decisions.
__global__ void moe_count_kernel(const int* __restrict__ topk_idx, int n, int E, int* __restrict__ counts) {
  __shared__ int h[256];
  for (int i = threadIdx.x; i < E; i += blockDim.x) h[i] = 0;
  __syncthreads();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int e = topk_idx[i];
    if (e >= 0 && e < E) atomicAdd(&h[e], 1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < E; i += blockDim.x)
    if (h[i]) atomicAdd(&counts[i], h[i]);
}

struct PeerPtrs { void* p[RB_MAX_RANKS]; };

// Publish this rank's histogram as row `rank` of the [world, E] count matrix on every rank (peer stores).
__global__ void moe_publish_counts_kernel(const int* __restrict__ counts, PeerPtrs counts_all, int rank, int world, int E) {
  const int r = blockIdx.x;
  if (r >= world) return;
  int* dst = reinterpret_cast<int*>(counts_all.p[r]) + (long long)rank * E;
  for (int i = threadIdx.x; i < E; i += blockDim.x) dst[i] = counts[i];
}

// Where this rank's rows for expert e start in the owner's expert-ordered receive buffer: the rows of the owner's
// lower experts (from all ranks) plus the rows of lower source ranks for e. Written to cursor[E + e].
__global__ void moe_send_base_kernel(const int* __restrict__ counts_all, int world, int E, int rank, int* __restrict__ cursor) {
  const int epr = E / world;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int owner = e / epr;
    int off = 0;
    for (int ee = owner * epr; ee < e; ++ee)
      for (int r = 0; r < world; ++r) off += counts_all[r * E + ee];
    for (int r = 0; r < rank; ++r) off += counts_all[r * E + e];
    cursor[E + e] = off;
  }
}

// Dispatch: row (t, j) goes to the owner of its expert. Position inside the owner's
// expert-ordered buffer = expert block offset on the owner + rows from lower source ranks +
// a running cursor for this (source, expert). ret_addr records where the result row must be
// written (this rank's y buffer, slot t*k+j), as seen from the owner.
__global__ void moe_permute_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ topk_idx, int T, int k,
                                   int d, int E, int world, int rank, const int* __restrict__ counts_all,
                                   int* __restrict__ cursor /*[2E]: running index | send base*/, PeerPtrs xp /*[cap, d] per rank*/,
                                   PeerPtrs ret_code /*u64[cap] per rank*/, int cap, int* status) {
  const int lane = threadIdx.x & 31;
  const long long gw = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (gw >= (long long)T * k) return;
  const int t = (int)(gw / k);
  const int e = topk_idx[gw];
  if (e < 0 || e >= E) { set_status(status, ST_BAD_INDEX); return; }
  const int epr = E / world;
  const int owner = e / epr;
  int pos = 0;
  if (lane == 0) pos = cursor[E + e] + atomicAdd(&cursor[e], 1);   // base of (this rank, e) on the owner + running index
  pos = __shfl_sync(0xffffffffu, pos, 0);
  if (pos >= cap) { set_status(status, ST_BAD_INDEX); return; }
  const uint4* src = reinterpret_cast<const uint4*>(x + (long long)t * d);
  uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(xp.p[owner]) + (long long)pos * d);
  for (int v = lane; v < (d >> 3); v += 32) dst[v] = src[v];
  if (lane == 0) {
    // home of the result: (source rank, slot t*k+j); the owner turns it into an address in ITS
    // mapping of the source's y buffer (peer mappings differ between processes)
    reinterpret_cast<unsigned long long*>(ret_code.p[owner])[pos] =
        ((unsigned long long)rank << 40) | (unsigned long long)gw;
  }
}

// Owner side: (source rank, slot) -> address of y[slot] in the source's buffer as mapped here.
__global__ void moe_translate_kernel(unsigned long long* __restrict__ ret, int n, PeerPtrs y_ptrs, int world, int d) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const unsigned long long code = ret[i];
    int src = (int)(code >> 40);
    if (src < 0 || src >= world) src = 0;
    const unsigned long long slot = code & ((1ull << 40) - 1);
    ret[i] = reinterpret_cast<unsigned long long>(y_ptrs.p[src]) + slot * (unsigned long long)d * 2ull;
  }
}

// out[t] (+)= sum_j w[t,j] * y[t*k+j]
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const float* __restrict__ w, int T, int k, int d,
                                   __nv_bfloat16* __restrict__ out, int accumulate) {
  const long long nvec = (long long)T * (d >> 3);
  const int vpr = d >> 3;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vpr;
    const int c = (int)(i % vpr) * 8;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (accumulate) {
      const uint4 o = *reinterpret_cast<const uint4*>(out + t * d + c);
      float2 f;
      f = unpack_bf16x2(o.x); acc[0] = f.x; acc[1] = f.y;
      f = unpack_bf16x2(o.y); acc[2] = f.x; acc[3] = f.y;
      f = unpack_bf16x2(o.z); acc[4] = f.x; acc[5] = f.y;
      f = unpack_bf16x2(o.w); acc[6] = f.x; acc[7] = f.y;
    }
    for (int j = 0; j < k; ++j) {
      const float wj = w[t * k + j];
      const uint4 v = __ldcg(reinterpret_cast<const uint4*>(y + (t * k + j) * d + c));
      float2 f;
      f = unpack_bf16x2(v.x); acc[0] += wj * f.x; acc[1] += wj * f.y;
      f = unpack_bf16x2(v.y); acc[2] += wj * f.x; acc[3] += wj * f.y;
      f = unpack_bf16x2(v.z); acc[4] += wj * f.x; acc[5] += wj * f.y;
      f = unpack_bf16x2(v.w); acc[6] += wj * f.x; acc[7] += wj * f.y;
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + t * d + c) = o;
  }
}


// ------------------------------------------------------------------------------------------------------------------
// Training: expert-grouped rows with every group padded to a multiple of 64 rows (zero rows), so that the weight
// gradient dW_e = dY_e^T X_e can run as one grouped launch whose K range is the group's row range: a 64-row k-block
// never straddles two experts. Everything is derived from the per-expert counts on the device (no host sync), and
// the row order inside an expert is the token order, so results do not depend on scheduling.

struct TrainTableDesc {
  int mode;        // 0 forward {a_row0, valid_rows, e * b_stride + n0, n0}; 1 data gradient {a_row0, valid_rows, e * b_stride, n0};
                   // 2 weight gradient {row0, rows, e, (m tile << 16) | n tile}
  int n_total;     // output columns per expert
  int bn;          // tile width
  int b_stride;    // rows of the stacked B matrix per expert (modes 0, 1); output rows per expert M (mode 2)
  int4* tiles;
  int* ntiles;
};
constexpr int MAX_TRAIN_TABLES = 6;
struct TrainTables { TrainTableDesc t[MAX_TRAIN_TABLES]; int n; };

// One CTA per table (blockIdx.x) plus every CTA's own copy of the offsets. offsets[e] = first row of expert e,
// offsets[E] = rows in use (all multiples of 64; an expert without tokens still gets 64 zero rows, which keeps its weight
// gradient an ordinary tile whose product is zero).
__global__ void moe_train_plan_kernel(const int* __restrict__ counts, int E, int* __restrict__ offsets, TrainTables tabs,
                                      int max_tiles, int cap_rows, int* __restrict__ status) {
  __shared__ int off_s[257];
  __shared__ int base_s[257];
  const TrainTableDesc d = tabs.t[blockIdx.x];
  const int nt = (d.n_total + d.bn - 1) / d.bn;
  // padded row counts and tile counts per expert, then two serial prefix sums over at most 256 entries
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int c = counts[e];
    off_s[e + 1] = c > 0 ? ((c + 63) / 64) * 64 : 64;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int o = 0, b = 0;
    off_s[0] = 0;
    for (int e = 0; e < E; ++e) {
      const int rows = off_s[e + 1];
      base_s[e] = b;
      b += (d.mode == 2 ? (d.b_stride + 127) / 128 : (rows + 127) / 128) * nt;
      o += rows;
      off_s[e + 1] = o;
    }
    base_s[E] = b;
    if (o > cap_rows || b > max_tiles) {
      set_status(status, ST_BAD_INDEX);
      base_s[E] = 0;
    }
    *d.ntiles = base_s[E];
  }
  __syncthreads();
  if (blockIdx.x == 0)
    for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = off_s[e];
  const int total = base_s[E];
  for (int t = threadIdx.x; t < total; t += blockDim.x) {
    int lo = 0, hi = E - 1;                       // the expert whose tile range holds t
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (base_s[mid] <= t) lo = mid; else hi = mid - 1;
    }
    const int e = lo, j = t - base_s[e];
    const int rows = off_s[e + 1] - off_s[e];
    const int mt = d.mode == 2 ? (d.b_stride + 127) / 128 : (rows + 127) / 128;
    // consecutive tiles share the B tile (modes 0, 1) or the A tile's k range (mode 2)
    const int in = j / mt, im = j % mt;
    int4 v;
    if (d.mode == 2) {
      v = make_int4(off_s[e], rows, e, (im << 16) | in);
    } else {
      const int r0 = off_s[e] + im * 128;
      v = make_int4(r0, min(128, off_s[e + 1] - r0), d.mode == 0 ? e * d.b_stride + in * d.bn : e * d.b_stride, in * d.bn);
    }
    d.tiles[t] = v;
  }
}

// One CTA per expert: walk the (token, slot) pairs in order and hand out the expert's rows in that order.
// row_of[i] = row of pair i; src_of[row] = pair of a row, -1 for the padding rows.
__global__ void moe_train_rows_kernel(const int* __restrict__ topk_idx, int n_pairs, const int* __restrict__ offsets,
                                      int* __restrict__ row_of, int* __restrict__ src_of) {
  const int e = blockIdx.x;
  const int row0 = offsets[e], row_end = offsets[e + 1];
  __shared__ int warp_sum[32];
  __shared__ int running;
  if (threadIdx.x == 0) running = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  for (int i0 = 0; i0 < n_pairs; i0 += blockDim.x) {
    const int i = i0 + threadIdx.x;
    const bool hit = i < n_pairs && topk_idx[i] == e;
    const unsigned m = __ballot_sync(0xffffffffu, hit);
    if (lane == 0) warp_sum[warp] = __popc(m);
    __syncthreads();
    int before = running;
    for (int w = 0; w < warp; ++w) before += warp_sum[w];
    if (hit) {
      const int row = row0 + before + __popc(m & ((1u << lane) - 1u));
      row_of[i] = row;
      src_of[row] = i;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int tot = 0;
      for (int w = 0; w < nwarp; ++w) tot += warp_sum[w];
      running += tot;
    }
    __syncthreads();
  }
  for (int r = row0 + running + threadIdx.x; r < row_end; r += blockDim.x) src_of[r] = -1;
}

// out[row] = scale(row) * src[src_of[row] / k] for the rows in use (zeros for padding rows); scale = w[src_of[row]] or 1.
__global__ void moe_train_gather_kernel(const __nv_bfloat16* __restrict__ src, const float* __restrict__ w,
                                        const int* __restrict__ src_of, const int* __restrict__ total_rows, int k, int d,
                                        __nv_bfloat16* __restrict__ out) {
  const int vpr = d >> 3;
  const long long nvec = (long long)(*total_rows) * vpr;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / vpr;
    const int c = (int)(i % vpr) * 8;
    const int s = src_of[row];
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (s >= 0) {
      v = *reinterpret_cast<const uint4*>(src + (long long)(s / k) * d + c);
      if (w != nullptr) {
        const float ws = w[s];
        float2 f;
        f = unpack_bf16x2(v.x); v.x = pack_bf16x2(ws * f.x, ws * f.y);
        f = unpack_bf16x2(v.y); v.y = pack_bf16x2(ws * f.x, ws * f.y);
        f = unpack_bf16x2(v.z); v.z = pack_bf16x2(ws * f.x, ws * f.y);
        f = unpack_bf16x2(v.w); v.w = pack_bf16x2(ws * f.x, ws * f.y);
      }
    }
    *reinterpret_cast<uint4*>(out + row * d + c) = v;
  }
}

// out[t] = sum_j (w ? w[t,j] : 1) * y[row_of[t*k+j]] (fp32 accumulation in slot order)
__global__ void moe_train_combine_kernel(const __nv_bfloat16* __restrict__ y, const float* __restrict__ w,
                                         const int* __restrict__ row_of, int T, int k, int d, __nv_bfloat16* __restrict__ out) {
  const int vpr = d >> 3;
  const long long nvec = (long long)T * vpr;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vpr;
    const int c = (int)(i % vpr) * 8;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < k; ++j) {
      const float wj = w != nullptr ? w[t * k + j] : 1.f;
      const uint4 v = *reinterpret_cast<const uint4*>(y + (long long)row_of[t * k + j] * d + c);
      float2 f;
      f = unpack_bf16x2(v.x); acc[0] += wj * f.x; acc[1] += wj * f.y;
      f = unpack_bf16x2(v.y); acc[2] += wj * f.x; acc[3] += wj * f.y;
      f = unpack_bf16x2(v.z); acc[4] += wj * f.x; acc[5] += wj * f.y;
      f = unpack_bf16x2(v.w); acc[6] += wj * f.x; acc[7] += wj * f.y;
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + t * d + c) = o;
  }
}

// dw[t,j] = <g[t,:], y[row_of[t*k+j],:]> : gradient of the combine weights. One warp per (token, slot).
__global__ void moe_train_dot_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ y,
                                     const int* __restrict__ row_of, int n_pairs, int k, int d, float* __restrict__ dw) {
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= n_pairs) return;
  const __nv_bfloat16* a = g + (long long)(i / k) * d;
  const __nv_bfloat16* b = y + (long long)row_of[i] * d;
  float acc = 0.f;
  for (int c = lane * 8; c < d; c += 256) {
    const uint4 va = *reinterpret_cast<const uint4*>(a + c), vb = *reinterpret_cast<const uint4*>(b + c);
    float2 fa, fb;
    fa = unpack_bf16x2(va.x); fb = unpack_bf16x2(vb.x); acc += fa.x * fb.x + fa.y * fb.y;
    fa = unpack_bf16x2(va.y); fb = unpack_bf16x2(vb.y); acc += fa.x * fb.x + fa.y * fb.y;
    fa = unpack_bf16x2(va.z); fb = unpack_bf16x2(vb.z); acc += fa.x * fb.x + fa.y * fb.y;
    fa = unpack_bf16x2(va.w); fb = unpack_bf16x2(vb.w); acc += fa.x * fb.x + fa.y * fb.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) dw[i] = acc;
}

}  // namespace rb

using namespace rb;
#define RB_OK() (cudaGetLastError() == cudaSuccess ? 0 : -11)
static PeerPtrs mk(void* const* p, int world) {
  PeerPtrs o;
  for (int i = 0; i < RB_MAX_RANKS; ++i) o.p[i] = i < world ? p[i] : nullptr;
  return o;
}

extern "C" int rb_moe_route(const float* logits, const float* bias, int T, int E, int k, int sigmoid_router,
                            int norm_topk, float scaling, int* topk_idx, float* topk_w, cudaStream_t s) {
  if (T <= 0) return 0;
  if (E > 32 * MAX_E_PER_LANE || k > 32 || k > E) return -1;
  moe_route_kernel<<<(T + 7) / 8, 256, 0, s>>>(logits, bias, T, E, k, sigmoid_router, norm_topk, scaling, topk_idx, topk_w, nullptr, 1, 1);
  return RB_OK();
}
// Routing plus the per-expert histogram of the choices (added into counts[E], which the caller zeroes).
extern "C" int rb_moe_route_count(const float* logits, const float* bias, int T, int E, int k, int sigmoid_router,
                                  int norm_topk, float scaling, int* topk_idx, float* topk_w, int* counts, cudaStream_t s) {
  if (T <= 0) return 0;
  if (E > 32 * MAX_E_PER_LANE || k > 32 || k > E || counts == nullptr) return -1;
  moe_route_kernel<<<(T + 7) / 8, 256, 0, s>>>(logits, bias, T, E, k, sigmoid_router, norm_topk, scaling, topk_idx, topk_w, counts, 1, 1);
  return RB_OK();
}
// The same with group-limited routing (n_group groups of E / n_group >= 2 experts, topk_group of them eligible).
// counts may be null (no histogram).
extern "C" int rb_moe_route_groups(const float* logits, const float* bias, int T, int E, int k, int norm_topk, float scaling,
                                   int n_group, int topk_group, int* topk_idx, float* topk_w, int* counts, cudaStream_t s) {
  if (T <= 0) return 0;
  if (E > 32 * MAX_E_PER_LANE || k > 32 || k > E) return -1;
  if (n_group < 1 || n_group > 32 || topk_group < 1 || topk_group > n_group || E % n_group != 0) return -1;
  if (n_group > 1 && E / n_group < 2) return -1;
  moe_route_kernel<<<(T + 7) / 8, 256, 0, s>>>(logits, bias, T, E, k, 1, norm_topk, scaling, topk_idx, topk_w, counts, n_group,
                                               topk_group);
  return RB_OK();
}
extern "C" int rb_moe_count(const int* topk_idx, int n, int E, int* counts, cudaStream_t s) {
  if (n <= 0) return 0;
  if (E > 256) return -1;
  int grid = (n + 255) / 256;
  if (grid > 148) grid = 148;
  moe_count_kernel<<<grid, 256, 0, s>>>(topk_idx, n, E, counts);
  return RB_OK();
}
extern "C" int rb_moe_publish_counts(const int* counts, void* const* counts_all, int rank, int world, int E, cudaStream_t s) {
  if (world <= 0 || world > RB_MAX_RANKS) return -1;
  moe_publish_counts_kernel<<<world, 128, 0, s>>>(counts, mk(counts_all, world), rank, world, E);
  return RB_OK();
}
extern "C" int rb_moe_plan(const int* counts_all, int world, int E, int e_lo, int e_hi, int* expert_offset, int n_gu,
                           int bn_gu, void* tiles_gu, int* ntiles_gu, int n_dn, int bn_dn, void* tiles_dn,
                           int* ntiles_dn, int max_tiles, int* status, cudaStream_t s) {
  if (e_hi - e_lo > 256 || e_hi <= e_lo) return -1;
  moe_plan_kernel<<<1, 256, 0, s>>>(counts_all, world, E, e_lo, e_hi, expert_offset, n_gu, bn_gu, (int4*)tiles_gu,
                                    ntiles_gu, n_dn, bn_dn, (int4*)tiles_dn, ntiles_dn, max_tiles, status, 0, nullptr);
  return RB_OK();
}
// The same plus the dispatch bases of rb_moe_permute_planned (cursor[E..2E)).
extern "C" int rb_moe_plan_dispatch(const int* counts_all, int world, int E, int e_lo, int e_hi, int* expert_offset, int n_gu,
                                    int bn_gu, void* tiles_gu, int* ntiles_gu, int n_dn, int bn_dn, void* tiles_dn,
                                    int* ntiles_dn, int max_tiles, int* status, int rank, int* cursor, cudaStream_t s) {
  if (e_hi - e_lo > 256 || e_hi <= e_lo || E % world != 0 || cursor == nullptr) return -1;
  moe_plan_kernel<<<1, 256, 0, s>>>(counts_all, world, E, e_lo, e_hi, expert_offset, n_gu, bn_gu, (int4*)tiles_gu,
                                    ntiles_gu, n_dn, bn_dn, (int4*)tiles_dn, ntiles_dn, max_tiles, status, rank, cursor);
  return RB_OK();
}
extern "C" int rb_moe_permute(const void* x, const int* topk_idx, int T, int k, int d, int E, int world, int rank,
                              const int* counts_all, int* cursor, void* const* xp_ptrs, void* const* ret_ptrs,
                              int cap, int* status, cudaStream_t s) {
  if (T <= 0) return 0;
  if (d % 8 != 0 || E % world != 0) return -1;
  const long long warps = (long long)T * k;
  moe_send_base_kernel<<<1, 256, 0, s>>>(counts_all, world, E, rank, cursor);
  moe_permute_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, s>>>((const __nv_bfloat16*)x, topk_idx, T, k, d, E, world, rank,
                                                                counts_all, cursor, mk(xp_ptrs, world), mk(ret_ptrs, world),
                                                                cap, status);
  return RB_OK();
}
// Dispatch when cursor[E..2E) already holds the send bases (rb_moe_plan_dispatch ran on the same counts).
extern "C" int rb_moe_permute_planned(const void* x, const int* topk_idx, int T, int k, int d, int E, int world, int rank,
                                      const int* counts_all, int* cursor, void* const* xp_ptrs, void* const* ret_ptrs,
                                      int cap, int* status, cudaStream_t s) {
  if (T <= 0) return 0;
  if (d % 8 != 0 || E % world != 0) return -1;
  const long long warps = (long long)T * k;
  moe_permute_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, s>>>((const __nv_bfloat16*)x, topk_idx, T, k, d, E, world, rank,
                                                                counts_all, cursor, mk(xp_ptrs, world), mk(ret_ptrs, world),
                                                                cap, status);
  return RB_OK();
}
extern "C" int rb_moe_translate(void* ret, int n, void* const* y_ptrs, int world, int d, cudaStream_t s) {
  if (n <= 0) return 0;
  int grid = (n + 255) / 256;
  if (grid > 148 * 4) grid = 148 * 4;
  moe_translate_kernel<<<grid, 256, 0, s>>>((unsigned long long*)ret, n, mk(y_ptrs, world), world, d);
  return RB_OK();
}
extern "C" int rb_moe_combine(const void* y, const float* w, int T, int k, int d, void* out, int accumulate,
                              cudaStream_t s) {
  if (T <= 0) return 0;
  const long long nvec = (long long)T * (d / 8);
  long long grid = (nvec + 255) / 256;
  if (grid > 148 * 8) grid = 148 * 8;
  moe_combine_kernel<<<(unsigned)grid, 256, 0, s>>>((const __nv_bfloat16*)y, w, T, k, d, (__nv_bfloat16*)out, accumulate);
  return RB_OK();
}

// ---------------------------------------------------------------- training (expert-grouped rows, padded to 64)
// tables: n_tables entries of {mode, n_total, bn, b_stride} in `desc` (4 ints each), output pointers in tiles / ntiles.
extern "C" int rb_moe_train_plan(const int* counts, int E, int* offsets, const int* desc, void* const* tiles, int* const* ntiles,
                                 int n_tables, int max_tiles, int cap_rows, int* status, cudaStream_t s) {
  if (E <= 0 || E > 256 || n_tables < 0 || n_tables > MAX_TRAIN_TABLES) return -1;
  TrainTables tabs;
  tabs.n = n_tables;
  for (int i = 0; i < n_tables; ++i) {
    tabs.t[i].mode = desc[4 * i]; tabs.t[i].n_total = desc[4 * i + 1]; tabs.t[i].bn = desc[4 * i + 2]; tabs.t[i].b_stride = desc[4 * i + 3];
    tabs.t[i].tiles = reinterpret_cast<int4*>(tiles[i]); tabs.t[i].ntiles = ntiles[i];
    if (tabs.t[i].mode < 0 || tabs.t[i].mode > 2 || tabs.t[i].bn <= 0 || tabs.t[i].n_total <= 0 || tabs.t[i].tiles == nullptr ||
        tabs.t[i].ntiles == nullptr)
      return -1;
    if (tabs.t[i].mode == 2 && ((tabs.t[i].b_stride + 127) / 128 > 0xffff || (tabs.t[i].n_total + tabs.t[i].bn - 1) / tabs.t[i].bn > 0xffff)) return -1;
  }
  if (n_tables == 0) return -1;
  moe_train_plan_kernel<<<n_tables, 256, 0, s>>>(counts, E, offsets, tabs, max_tiles, cap_rows, status);
  return RB_OK();
}

extern "C" int rb_moe_train_rows(const int* topk_idx, int n_pairs, int E, const int* offsets, int* row_of, int* src_of, cudaStream_t s) {
  if (n_pairs <= 0) return 0;
  moe_train_rows_kernel<<<E, 1024, 0, s>>>(topk_idx, n_pairs, offsets, row_of, src_of);
  return RB_OK();
}

extern "C" int rb_moe_train_gather(const void* src, const float* w, const int* src_of, const int* total_rows, int cap_rows, int k, int d,
                                   void* out, cudaStream_t s) {
  if (cap_rows <= 0) return 0;
  if (d % 8 != 0) return -1;
  long long grid = ((long long)cap_rows * (d / 8) + 255) / 256;
  if (grid > 148 * 8) grid = 148 * 8;
  moe_train_gather_kernel<<<(unsigned)grid, 256, 0, s>>>((const __nv_bfloat16*)src, w, src_of, total_rows, k, d, (__nv_bfloat16*)out);
  return RB_OK();
}

extern "C" int rb_moe_train_combine(const void* y, const float* w, const int* row_of, int T, int k, int d, void* out, cudaStream_t s) {
  if (T <= 0) return 0;
  if (d % 8 != 0) return -1;
  long long grid = ((long long)T * (d / 8) + 255) / 256;
  if (grid > 148 * 8) grid = 148 * 8;
  moe_train_combine_kernel<<<(unsigned)grid, 256, 0, s>>>((const __nv_bfloat16*)y, w, row_of, T, k, d, (__nv_bfloat16*)out);
  return RB_OK();
}

extern "C" int rb_moe_train_dot(const void* g, const void* y, const int* row_of, int n_pairs, int k, int d, float* dw, cudaStream_t s) {
  if (n_pairs <= 0) return 0;
  if (d % 8 != 0) return -1;
  moe_train_dot_kernel<<<(n_pairs + 7) / 8, 256, 0, s>>>((const __nv_bfloat16*)g, (const __nv_bfloat16*)y, row_of, n_pairs, k, d, dw);
  return RB_OK();
}
