// C[M, N] (bf16) = scale_a * scale_b * A[M, K] (e4m3) . W[N, K]^T (e4m3): the dense GEMM's pipeline (TMA-fed ring, one
// elected thread issuing tcgen05.mma, double-buffered TMEM accumulators) with kind::f8f6f4 instructions — twice the
// math per byte of the bf16 kernel. Per-tensor scales live in device memory (a quantiser writes them).
// kern_quant_e4m3: x (bf16) -> e4m3 bytes with one scale per tensor: scale = amax / 448 (two launches: amax, cast).
// Reference counterpart: the library call sites extern:cublaslt_fp8_tn (crates/kern-runtime/src/cublas.rs:387-505).
#define KERN_GEMM_NO_ENTRIES
#include "gemm_bf16.cu"

#include <cuda_fp8.h>

using namespace kern;

#define KERN_FP8_GEMM_ENTRY(name, BN, EPI)                                                                        \
  extern "C" __global__ void __launch_bounds__(192, 1)                                                            \
      name(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, void* C,          \
           const void* R, const float* scale_a, const float* scale_b, int M, int N, int K, int ldc, int* err) {    \
    kern::gemm_body<BN, EPI, false, true>(&tma_a, &tma_b, C, R, M, N, K, ldc, err, nullptr, nullptr,               \
                                          kern::ScatterArgs(), scale_a, scale_b);                                  \
  }

KERN_FP8_GEMM_ENTRY(kern_gemm_e4m3_tn_n256, 256, 0)
KERN_FP8_GEMM_ENTRY(kern_gemm_e4m3_tn_n128, 128, 0)
KERN_FP8_GEMM_ENTRY(kern_gemm_e4m3_tn_n64, 64, 0)
KERN_FP8_GEMM_ENTRY(kern_gemm_e4m3_tn_f32_n256, 256, 1)
KERN_FP8_GEMM_ENTRY(kern_gemm_e4m3_tn_f32_n128, 128, 1)
KERN_FP8_GEMM_ENTRY(kern_gemm_e4m3_tn_f32_n64, 64, 1)
KERN_FP8_GEMM_ENTRY(kern_gemm_e4m3_tn_acc_n256, 256, 2)
KERN_FP8_GEMM_ENTRY(kern_gemm_e4m3_tn_acc_n128, 128, 2)

// amax[0] = max |x| (as ordered float bits; zero it first). grid any, block 256.
extern "C" __global__ void kern_amax_bf16(const __nv_bfloat16* x, unsigned long long n, unsigned* amax_bits) {
  float m = 0.f;
  for (unsigned long long i = blockIdx.x * 256ull + threadIdx.x; i < n; i += (unsigned long long)gridDim.x * 256ull)
    m = fmaxf(m, fabsf(__bfloat162float(x[i])));
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) atomicMax(amax_bits, __float_as_uint(m));      // non-negative floats order as integers
}

// scale[0] = amax / 448 (1 when the tensor is all zero); y = e4m3(x / scale). grid any, block 256.
extern "C" __global__ void kern_quant_e4m3(const __nv_bfloat16* x, unsigned char* y, unsigned long long n,
                                           const unsigned* amax_bits, float* scale) {
  const float amax = __uint_as_float(amax_bits[0]);
  const float s = amax > 0.f ? amax / 448.f : 1.f;
  if (blockIdx.x == 0 && threadIdx.x == 0) scale[0] = s;
  const float inv = 1.f / s;
  for (unsigned long long i = blockIdx.x * 256ull + threadIdx.x; i < n; i += (unsigned long long)gridDim.x * 256ull)
    y[i] = (unsigned char)__nv_cvt_float_to_fp8(__bfloat162float(x[i]) * inv, __NV_SATFINITE, __NV_E4M3);
}
