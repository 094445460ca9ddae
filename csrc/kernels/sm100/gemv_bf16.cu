// C[M, N] = A[M, K] . W[N, K]^T for a handful of rows (decode steps of a few sequences): the weights are read once,
// straight from HBM with 16-byte loads, and every one of the 148 SMs streams its share — a 128-row tensor-core tile
// would leave most of the machine idle and most of the tile empty at these sizes. The op is bandwidth-bound: the
// roofline is the weight bytes over the copy bandwidth.
//
// A CTA owns four weight rows at a time (so A is fetched once per four outputs); its 256 threads stride over the K
// vectors of those rows, partial sums meet through shuffles and shared memory. Persistent grid: CTAs take row groups
// round-robin, eight or so resident per SM, so tens of kilobytes of loads are in flight on every SM.
// Epilogues as in the tensor-core GEMM: 0 store bf16, 1 store f32, 2 accumulate into a bf16 residual, 3 SwiGLU over
// weights stacked [gate rows ; up rows] (two gate rows and their two up rows per group).
// (The reference calls a library GEMM for every shape; this kernel has no counterpart there.)
#include "common.cuh"

using namespace kern;

namespace {

template <int MT, int EPI>
__device__ __forceinline__ void gemv_body(const __nv_bfloat16* A, const __nv_bfloat16* W, void* Cv, const void* Rv, int M,
                                          int N, int K, int lda, int ldc) {
  constexpr int R = 4;                       // weight rows per CTA per group
  __shared__ float part[8][MT * R];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv = K >> 3;
  const int half = N >> 1;
  const int groups = EPI == 3 ? (half + 1) / 2 : (N + R - 1) / R;
  for (int g = blockIdx.x; g < groups; g += gridDim.x) {
    int rows[R];
    if constexpr (EPI == 3) {
      rows[0] = 2 * g; rows[1] = 2 * g + 1; rows[2] = half + 2 * g; rows[3] = half + 2 * g + 1;
      if (rows[1] >= half) { rows[1] = rows[0]; rows[3] = rows[2]; }     // odd tail: duplicate, the store skips it
    } else {
#pragma unroll
      for (int r = 0; r < R; ++r) rows[r] = min(g * R + r, N - 1);
    }
    float acc[MT][R];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int r = 0; r < R; ++r) acc[m][r] = 0.f;
    const uint4* w0 = reinterpret_cast<const uint4*>(W + (size_t)rows[0] * K);
    const uint4* w1 = reinterpret_cast<const uint4*>(W + (size_t)rows[1] * K);
    const uint4* w2 = reinterpret_cast<const uint4*>(W + (size_t)rows[2] * K);
    const uint4* w3 = reinterpret_cast<const uint4*>(W + (size_t)rows[3] * K);
    // the whole CTA strides over the K vectors of its four rows: 256 x 4 x 16 bytes in flight per pass
#pragma unroll 2
    for (int v = threadIdx.x; v < kv; v += 256) {
      uint4 wv[R];
      wv[0] = __ldcs(w0 + v); wv[1] = __ldcs(w1 + v); wv[2] = __ldcs(w2 + v); wv[3] = __ldcs(w3 + v);   // streamed once
      float wf[R][8];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        float2 a = unpack_bf16x2(wv[r].x), b = unpack_bf16x2(wv[r].y), c = unpack_bf16x2(wv[r].z), d = unpack_bf16x2(wv[r].w);
        wf[r][0] = a.x; wf[r][1] = a.y; wf[r][2] = b.x; wf[r][3] = b.y; wf[r][4] = c.x; wf[r][5] = c.y; wf[r][6] = d.x; wf[r][7] = d.y;
      }
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        if (m < M) {
          const uint4 av = __ldg(reinterpret_cast<const uint4*>(A + (size_t)m * lda) + v);
          float2 a = unpack_bf16x2(av.x), b = unpack_bf16x2(av.y), c = unpack_bf16x2(av.z), d = unpack_bf16x2(av.w);
          const float af[8] = {a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y};
#pragma unroll
          for (int r = 0; r < R; ++r)
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[m][r] += af[e] * wf[r][e];
        }
      }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float s = warp_sum(acc[m][r]);
        if (lane == 0) part[warp][m * R + r] = s;
      }
    __syncthreads();
    if (threadIdx.x < MT * R) {
      const int m = threadIdx.x / R, r = threadIdx.x % R;
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) s += part[w][threadIdx.x];
      part[0][threadIdx.x] = s;            // column threadIdx.x is only read by this thread above
      (void)m; (void)r;
    }
    __syncthreads();
    if (threadIdx.x < MT * R) {
      const int m = threadIdx.x / R, r = threadIdx.x % R;
      if (m < M) {
        if constexpr (EPI == 3) {
          // outputs 2g (r = 0) and 2g + 1 (r = 1): gate in columns 0..1, up in 2..3
          if (r < 2 && 2 * g + r < half)
            reinterpret_cast<__nv_bfloat16*>(Cv)[(size_t)m * ldc + 2 * g + r] =
                __float2bfloat16(silu(part[0][m * R + r]) * part[0][m * R + 2 + r]);
        } else {
          const int n = g * R + r;
          if (n < N) {
            const float v = part[0][threadIdx.x];
            if constexpr (EPI == 1) {
              reinterpret_cast<float*>(Cv)[(size_t)m * ldc + n] = v;
            } else if constexpr (EPI == 2) {
              const float res = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(Rv)[(size_t)m * ldc + n]);
              reinterpret_cast<__nv_bfloat16*>(Cv)[(size_t)m * ldc + n] = __float2bfloat16(v + res);
            } else {
              reinterpret_cast<__nv_bfloat16*>(Cv)[(size_t)m * ldc + n] = __float2bfloat16(v);
            }
          }
        }
      }
    }
    __syncthreads();     // `part` is reused by the next group
  }
}

}  // namespace

#define KERN_GEMV_ENTRY(name, MT, EPI)                                                                              \
  extern "C" __global__ void __launch_bounds__(256)                                                                 \
      name(const __nv_bfloat16* A, const __nv_bfloat16* W, void* C, const void* R, int M, int N, int K, int lda,     \
           int ldc, int* err) {                                                                                      \
    pdl_wait();                                                                                                      \
    if (M > MT) {                                                                                                    \
      if (threadIdx.x == 0 && blockIdx.x == 0) set_error(err, ERR_BOUNDS);   /* more rows than this variant holds */  \
      return;                                                                                                        \
    }                                                                                                                \
    gemv_body<MT, EPI>(A, W, C, R, M, N, K, lda, ldc);                                                               \
  }

#define KERN_GEMV_FAMILY(MT)                                       \
  KERN_GEMV_ENTRY(kern_gemv_bf16_tn_m##MT, MT, 0)                  \
  KERN_GEMV_ENTRY(kern_gemv_bf16_tn_f32_m##MT, MT, 1)              \
  KERN_GEMV_ENTRY(kern_gemv_bf16_tn_acc_m##MT, MT, 2)              \
  KERN_GEMV_ENTRY(kern_gemv_bf16_tn_swiglu_m##MT, MT, 3)

KERN_GEMV_FAMILY(1)
KERN_GEMV_FAMILY(2)
KERN_GEMV_FAMILY(4)
KERN_GEMV_FAMILY(8)
