// C ABI of the sm_100a bf16 GEMM (tcgen05 / TMEM / TMA). Mirrored field by field by the
// ctypes structure in research_b200/ops/gemm.py.
#pragma once
#include <cuda_runtime.h>

#define RB_MAX_PARTS 8

// epilogue modes
#define RB_EPI_STORE 0            // C = acc (+bias) (+residual), local store
#define RB_EPI_REDUCE_SCATTER 1   // sum over ranks, rank r keeps row slab r
#define RB_EPI_ALL_REDUCE 2       // sum over ranks, every rank receives all rows
// One-shot all-reduce for small outputs (decode): every rank pushes its partial tile to EVERY rank's
// staging slab [src][M][N] and then sums all sources for the tiles it computed, writing only its own
// output. One cross-GPU hop, no ownership, no trailing barrier; traffic grows with the rank count.
#define RB_EPI_ALL_REDUCE_ONESHOT 3

#ifdef __cplusplus
extern "C" {
#endif

typedef struct RbGemmArgs {
  const void* A[RB_MAX_PARTS];   // row slab i of A (may be another GPU's memory)
  const void* B[RB_MAX_PARTS];   // row slab i of B (may be another GPU's memory)
  void* C;
  const void* bias;              // bf16 [N] or NULL
  const void* residual;          // bf16 [M, ldr] or NULL
  long long lda, ldb, ldc, ldr;  // leading dimensions in elements
  int M, N, K;
  int a_parts, b_parts;
  int a_mn_major, b_mn_major;
  int out_f32;
  int bn;                        // 0 = choose; else 32/64/128/256
  int max_ctas;                  // 0 = one per SM
  int epi_mode;
  int rank, world;
  const int* a_ready;            // optional [a_parts] flags, waited for >= ready_epoch
  const int* b_ready;            // optional [b_parts]
  int ready_epoch;
  int reduce_epoch;
  void* stage_ptrs[RB_MAX_PARTS];
  int* flag_ptrs[RB_MAX_PARTS];
  void* out_ptrs[RB_MAX_PARTS];
  int* status;                   // device int, 0 = ok, else rb::StatusCode
  // Reduce modes under CUDA-graph replay: when epoch_counter is set the kernel uses
  // epoch = *epoch_counter + 1 (the last CTA to finish stores it back), and picks the staging /
  // flag slab by epoch parity, so a captured launch stays correct on every replay.
  int* epoch_counter;
  int* cta_ticket;
  long long stage_parity_bytes;
  long long flag_parity_bytes;
  // Grouped mode (mixture of experts): tiles come from a device table of int4
  // {a_row0, valid_rows, b_row0, n0}; *num_tiles_ptr entries. A is [rows, K], B is
  // [groups * group_n, K] (group_n output columns per group), C row = A row. When row_dst is
  // set, output row r is written to the address row_dst[r] (possibly another GPU's memory)
  // instead of C: the combine of expert-parallel MoE fused into the epilogue.
  const int* tile_table;
  const int* num_tiles_ptr;
  int group_n;
  int max_tiles;
  const unsigned long long* row_dst;
  // Fused SwiGLU epilogue: B holds gate and up rows interleaved in blocks of bn/2 (block j =
  // gate rows [j*bn/2, (j+1)*bn/2) followed by the matching up rows); the kernel writes
  // silu(gate) * up to C, which has N/2 columns. Requires an explicit bn and N % bn == 0.
  int swiglu;
  // Split-K for skinny problems (few output tiles, long K): the K loop of every tile is cut
  // into split_k slices computed by different CTAs; each writes an fp32 partial tile to
  // splitk_ws [split_k][M][N] and the last CTA to finish a tile (ticket counter, self-resetting)
  // sums the slices in fixed order and applies the epilogue. Deterministic.
  int split_k;
  float* splitk_ws;
  int* splitk_tickets;           // [tiles], zero before first use
  // Scaled epilogue C = alpha * (A B^T) + bias + beta * residual (used when scaled_epilogue != 0).
  int scaled_epilogue;
  float alpha, beta;
  // Symmetric output (C = A A^T and friends): after the normal store every element below the
  // diagonal is also written to its transposed position, so a tile table that lists only the tiles
  // touching the lower triangle produces the full matrix.
  int mirror;
  // 8-bit floating point operands (both K-major): bit 0 enables, bit 1 = A is e5m2, bit 2 = B is
  // e5m2 (otherwise e4m3). The caller describes the operands as if they were bf16 matrices with half
  // as many columns (K, lda, ldb in units of two bytes): the tiles are moved as bytes and only the
  // tensor-core instruction differs. Per-tensor scales go into alpha.
  int fp8;
  // Fused sampling epilogue (lm_head): instead of storing the fp32 logits, every tile reduces its
  // columns per row to (running max, sum of exponentials, best Gumbel-perturbed score, the logit and
  // column of that score) and writes the 8-float record sample_ws[row][n_tile]; rb_sample_merge
  // finishes token and log-probability. Same random stream as rb_sample_logprob.
  float* sample_ws;
  const float* sample_temperature;              // [M]
  const unsigned long long* sample_seeds;       // [M]
  const unsigned long long* sample_step_ptr;    // device step counter (may be null)
  unsigned long long sample_step_add;
  // Split-K inside a thread-block cluster (split_k = 2, 4 or 8 CTAs per cluster): the slices exchange their fp32
  // partial tiles through distributed shared memory and each CTA finishes one column slice of the tile. Needs no
  // workspace or tickets; bn / split_k must be at least 8 columns. Deterministic.
  int cluster_split;
  // Folded RMSNorm: C = rstd(row) * (A B^T) (+bias, SwiGLU), rstd = rsqrt(mean(A[row,:]^2) + norm_eps), computed
  // inside the kernel from the A tiles as they stream through shared memory. The caller multiplies the norm weight
  // into B's columns beforehand. K-major A, plain store or SwiGLU epilogue, no split.
  int norm_fold;
  float norm_eps;
  // Fused all-gather (sharded parameters): the launch also copies `gather_parts` equal, contiguous blocks of
  // gather_part_bytes from gather_src[r] (rank r's shard; peer memory, plain loads) to gather_dst + r * bytes in local
  // memory, this rank's own part first, and publishes gather_ready[r] = gather_epoch when part r is complete
  // (gather_count: [parts] counters, zero between launches). To consume the gathered matrix in the SAME launch
  // describe it as the B operand with b_parts = gather_parts, B[r] = gather_dst + r * bytes, b_ready = gather_ready,
  // ready_epoch = gather_epoch and b_part_rot = rank: tiles of a part start when that part has landed. A launch
  // whose operands are unrelated (a weight-gradient GEMM) can carry the gather for the launch that follows it.
  const void* gather_src[RB_MAX_PARTS];
  void* gather_dst;
  long long gather_part_bytes;
  int* gather_count;
  int* gather_ready;
  int gather_epoch;
  int gather_parts;
  int b_part_rot;                // visit B's parts starting at this one
  // Ready epoch of a_ready / b_ready read from device memory at kernel start instead of ready_epoch: a launch
  // captured in a CUDA graph then waits for the epoch its own replay's signal kernel published.
  const int* ready_epoch_ptr;
  // Gather of shards that the peers produce just before the launch (tensor-parallel activations): a gather warp
  // waits for gather_src_ready[r] >= the ready epoch before copying part r (the own part needs no wait). With
  // gather_wait_all the gathered matrix is the launch's A operand as one matrix (A[0] = gather_dst, a_parts = 1)
  // and the tile producer waits for every part; the gather epoch is then the ready epoch too, so a launch captured
  // in a CUDA graph (ready_epoch_ptr) publishes a fresh value on every replay.
  const int* gather_src_ready;
  int gather_wait_all;
  // Grouped mode for the backward pass of a mixture of experts (tile_table set). 0: the forward form above.
  // 1 (data gradient): B is MN-major, the groups' [group K, N] matrices stacked along its rows (group_b_rows rows in
  // all); table entries are {a_row0, valid_rows, first B row of the group, n0} and K is the K extent of one group.
  // 2 (weight gradient): A [rows, M] and B [rows, N] are both MN-major and the contraction runs over a group's row
  // range; table entries are {first row, row count (a multiple of 64), group, (m tile << 16) | n tile}, the output of
  // group g is C rows [g * M, (g + 1) * M), and K is the total row count of A and B.
  int group_mode;
  int group_b_rows;
} RbGemmArgs;

// Token and log-probability from the per-tile records written by the sampling epilogue.
int rb_sample_merge(const float* sample_ws, int M, int n_tiles, int* out_tokens, float* out_logprobs,
                    cudaStream_t stream);

int rb_gemm_bf16_ex(const RbGemmArgs* args, cudaStream_t stream);

int rb_gemm_bf16(const void* A, const void* B, void* C, const void* bias, const void* residual,
                 int M, int N, int K, long long lda, long long ldb, long long ldc, long long ldr,
                 int a_mn_major, int b_mn_major, int out_f32, int bn, int* status,
                 cudaStream_t stream);

#ifdef __cplusplus
}
#endif
