// Low-precision kernels for sm_100a.
//
// rb_nvfp4_gemv: block-scaled FP4 matrix-vector product
//     c[l, m] = sum_k  a[l, m, k] * sfa[l, m, k/16] * b[l, k] * sfb[l, k/16]        (fp16 result)
// a, b hold two e2m1 values per byte (low nibble first), sfa / sfb are e4m3 bytes, one per 16
// elements, all row-major with k fastest (the plain layout of dev/kernels-gpumode/nvfp4/
// reference_kernel.py:29-55, which feeds the same numbers to a block-scaled tensor-core GEMM with N
// padded to 128). A matrix-vector product has no operand reuse for a tensor core to exploit, so the
// kernel is a bandwidth design: one warp per row, 16-byte loads of a (32 values = two scale blocks
// per lane and step), b decoded once per CTA into shared memory as half2, e2m1 pairs converted with the
// sm_100a `cvt.rn.f16x2.e2m1x2` instruction and multiplied with HFMA2 (sums of four exact products stay
// exact in fp16), block sums scaled and accumulated in fp32, one shuffle reduction per row.
#include "common.cuh"

#include <cuda_fp16.h>

namespace rb {

// e2m1 nibble -> value * 2^-14 as fp32 (the nibble's exponent/mantissa bits dropped into an fp16).
__device__ __forceinline__ float e2m1_raw(uint32_t nib) {
  const unsigned short h = (unsigned short)(((nib & 7u) << 9) | ((nib & 8u) << 12));
  return __half2float(__ushort_as_half(h));
}
// e4m3 byte -> value * 2^-8 as fp32.
__device__ __forceinline__ float e4m3_raw(uint32_t byte) {
  const unsigned short h = (unsigned short)(((byte & 0x7fu) << 7) | ((byte & 0x80u) << 8));
  return __half2float(__ushort_as_half(h));
}

constexpr int GEMV_WARPS = 4;

// One byte (two e2m1 values) -> half2 with the sm_100a conversion instruction. Both operands of the
// dot product go through the same instruction, so which nibble lands in which half does not matter.
__device__ __forceinline__ __half2 e2m1x2_to_half2(uint32_t byte) {
  uint32_t d;
  asm("{\n\t.reg .b8 t;\n\tcvt.u8.u32 t, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, t;\n\t}" : "=r"(d) : "r"(byte));
  return *reinterpret_cast<__half2*>(&d);
}

// R rows per warp: the R row loads of a step are independent (memory-level parallelism) and share
// the b fragments read from shared memory; a CTA covers GEMV_WARPS * R rows per decode of b.
template <int R>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
nvfp4_gemv_kernel(const uint8_t* __restrict__ a, const uint8_t* __restrict__ b, const uint8_t* __restrict__ sfa,
                  const uint8_t* __restrict__ sfb, __half* __restrict__ c, int M, int K) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int l = blockIdx.y;
  const int kb = K / 2, ks = K / 16;                 // bytes of data / scales per row
  __half2* b_s = reinterpret_cast<__half2*>(smem);    // [K/2] decoded pairs of b
  float* sfb_s = reinterpret_cast<float*>(smem + (size_t)kb * 4);   // [K/16] decoded (value * 2^-8)
  pdl_launch_dependents();
  pdl_wait();
  const uint8_t* bl = b + (long long)l * kb;
  for (int i = threadIdx.x; i < kb; i += blockDim.x) b_s[i] = e2m1x2_to_half2(bl[i]);
  for (int i = threadIdx.x; i < ks; i += blockDim.x) sfb_s[i] = e4m3_raw(sfb[(long long)l * ks + i]);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = (blockIdx.x * GEMV_WARPS + warp) * R;
  if (row0 >= M) return;
  const uint8_t* ar[R];
  const uint8_t* sr[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int row = min(row0 + r, M - 1);             // rows past the end recompute the last row, unused
    ar[r] = a + ((long long)l * M + row) * kb;
    sr[r] = sfa + ((long long)l * M + row) * ks;
  }
  float acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = 0.f;
  for (int chunk = lane; chunk * 16 < kb; chunk += 32) {          // 16 bytes = 32 values = 2 scale blocks
    uint4 av[R];
    unsigned short s2[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      av[r] = __ldg(reinterpret_cast<const uint4*>(ar[r] + chunk * 16));
      s2[r] = __ldg(reinterpret_cast<const unsigned short*>(sr[r] + chunk * 2));
    }
    const uint4* bq = reinterpret_cast<const uint4*>(b_s + chunk * 16);
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
      const uint4 b0 = bq[blk * 2], b1 = bq[blk * 2 + 1];
      const __half2 bh[8] = {*reinterpret_cast<const __half2*>(&b0.x), *reinterpret_cast<const __half2*>(&b0.y),
                             *reinterpret_cast<const __half2*>(&b0.z), *reinterpret_cast<const __half2*>(&b0.w),
                             *reinterpret_cast<const __half2*>(&b1.x), *reinterpret_cast<const __half2*>(&b1.y),
                             *reinterpret_cast<const __half2*>(&b1.z), *reinterpret_cast<const __half2*>(&b1.w)};
      const float sb = sfb_s[chunk * 2 + blk];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const uint32_t x0 = blk == 0 ? av[r].x : av[r].z, x1 = blk == 0 ? av[r].y : av[r].w;
        // 8 bytes of a against 8 half2 of b; each half2 lane adds 4 exact products (|sum| <= 144)
        __half2 p0 = __hmul2(e2m1x2_to_half2(x0 & 0xffu), bh[0]);
        __half2 p1 = __hmul2(e2m1x2_to_half2((x0 >> 8) & 0xffu), bh[1]);
        p0 = __hfma2(e2m1x2_to_half2((x0 >> 16) & 0xffu), bh[2], p0);
        p1 = __hfma2(e2m1x2_to_half2(x0 >> 24), bh[3], p1);
        p0 = __hfma2(e2m1x2_to_half2(x1 & 0xffu), bh[4], p0);
        p1 = __hfma2(e2m1x2_to_half2((x1 >> 8) & 0xffu), bh[5], p1);
        p0 = __hfma2(e2m1x2_to_half2((x1 >> 16) & 0xffu), bh[6], p0);
        p1 = __hfma2(e2m1x2_to_half2(x1 >> 24), bh[7], p1);
        const float2 f0 = __half22float2(p0), f1 = __half22float2(p1);
        acc[r] = fmaf((f0.x + f0.y) + (f1.x + f1.y), e4m3_raw((s2[r] >> (8 * blk)) & 0xffu) * sb, acc[r]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float v = acc[r];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    // undo the scale decode: 2^8 per e4m3 factor
    if (lane == 0 && row0 + r < M) c[(long long)l * M + row0 + r] = __float2half_rn(v * 65536.f);
  }
}

template <int R>
static int launch_gemv(const void* a, const void* b, const void* sfa, const void* sfb, void* c, int L, int M, int K,
                       int smem, cudaStream_t stream) {
  static int attr_smem = 48 * 1024;
  if (smem > attr_smem) {
    if (cudaFuncSetAttribute(nvfp4_gemv_kernel<R>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -10;
    attr_smem = smem;
  }
  dim3 grid((M + GEMV_WARPS * R - 1) / (GEMV_WARPS * R), L);
  return launch_kernel(nvfp4_gemv_kernel<R>, grid, dim3(GEMV_WARPS * 32), smem, stream, (const uint8_t*)a, (const uint8_t*)b,
                       (const uint8_t*)sfa, (const uint8_t*)sfb, (__half*)c, M, K) == cudaSuccess ? 0 : -11;
}

}  // namespace rb

extern "C" {

// a [L, M, K/2], b [L, K/2], sfa [L, M, K/16], sfb [L, K/16] bytes; c [L, M] fp16. K % 32 == 0.
int rb_nvfp4_gemv(const void* a, const void* b, const void* sfa, const void* sfb, void* c, int L, int M, int K,
                  cudaStream_t stream) {
  using namespace rb;
  if (L <= 0 || M <= 0) return 0;
  if (K <= 0 || K % 32 != 0) return -1;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) return -2;
  const int smem = (K / 2) * 4 + (K / 16) * 4;   // b as half2 per byte + decoded scales
  if (smem > 200 * 1024) return -3;
  // small problems: one row per warp (more CTAs); large ones: four rows per warp (more loads in flight)
  const long long rows = (long long)L * M;
  const int rc = rows >= 2048 ? launch_gemv<4>(a, b, sfa, sfb, c, L, M, K, smem, stream)
                                                    : launch_gemv<1>(a, b, sfa, sfb, c, L, M, K, smem, stream);
  if (rc != 0) return rc;
  return cudaGetLastError() == cudaSuccess ? 0 : -12;
}

}  // extern "C"
