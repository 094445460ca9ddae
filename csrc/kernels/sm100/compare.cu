// A/B comparison on the device, so a test never copies two whole buffers to the host to learn they are equal.
//   kern_cmp_reduce      element-wise comparison of two buffers of one dtype -> 6 u64:
//                        [differing, signed-zero-only, nan-on-one-side, measured, max ulp distance, max |a-b| bits (f64)]
//   kern_changed_blocks  bitmap of the 64-byte blocks in which `pre` and `post` differ (what a span wrote)
//   kern_logit_rows      per logits row: arg-max of both sides, top-1 margin of A, KL(A || B) -> 4 u64
// dtype codes: 0 bf16, 1 f16, 2 f32, 3 bytes (compared as u8, ulp = |a - b|).
// Reference counterpart: crates/kern-runtime/src/compare.cu:125 (cmp_reduce), :143 (changed_blocks), :207 (logit_rows).
#include <cuda_fp16.h>

#include "common.cuh"

using namespace kern;

namespace {
__device__ __forceinline__ float load_as_f32(const uint8_t* p, size_t i, int dtype, long long& ordered) {
  if (dtype == 0) {
    const unsigned short b = reinterpret_cast<const unsigned short*>(p)[i];
    ordered = (b & 0x8000) ? -(long long)(b & 0x7fff) : (long long)b;
    return __uint_as_float((unsigned)b << 16);
  }
  if (dtype == 1) {
    const unsigned short b = reinterpret_cast<const unsigned short*>(p)[i];
    ordered = (b & 0x8000) ? -(long long)(b & 0x7fff) : (long long)b;
    return __half2float(reinterpret_cast<const __half*>(p)[i]);
  }
  if (dtype == 2) {
    const unsigned b = reinterpret_cast<const unsigned*>(p)[i];
    ordered = (b & 0x80000000u) ? -(long long)(b & 0x7fffffffu) : (long long)b;
    return __uint_as_float(b);
  }
  ordered = p[i];
  return (float)p[i];
}
}  // namespace

extern "C" __global__ void __launch_bounds__(256)
    kern_cmp_reduce(const uint8_t* a, const uint8_t* b, unsigned long long n, int dtype, unsigned long long* out) {
  unsigned long long n_diff = 0, zero = 0, nan_one = 0, measured = 0, max_ulp = 0;
  double max_abs = 0.0;
  for (unsigned long long i = blockIdx.x * 256ull + threadIdx.x; i < n; i += (unsigned long long)gridDim.x * 256ull) {
    long long oa, ob;
    const float fa = load_as_f32(a, i, dtype, oa), fb = load_as_f32(b, i, dtype, ob);
    const bool na = fa != fa, nb = fb != fb;
    if (na && nb) continue;                                       // NaN on both sides counts as equal
    if (na != nb) { ++n_diff; ++nan_one; continue; }
    if (fa == 0.f && fb == 0.f) {                                 // +0 vs -0: noted, not a difference
      if (signbit(fa) != signbit(fb)) ++zero;
      continue;
    }
    if (oa == ob) continue;
    ++n_diff; ++measured;
    const unsigned long long ulp = (unsigned long long)(oa > ob ? oa - ob : ob - oa);
    max_ulp = ulp > max_ulp ? ulp : max_ulp;
    const double d = fabs((double)fa - (double)fb);
    max_abs = d > max_abs ? d : max_abs;
  }
  for (int o = 16; o > 0; o >>= 1) {
    n_diff += __shfl_xor_sync(0xffffffffu, n_diff, o);
    zero += __shfl_xor_sync(0xffffffffu, zero, o);
    nan_one += __shfl_xor_sync(0xffffffffu, nan_one, o);
    measured += __shfl_xor_sync(0xffffffffu, measured, o);
    const unsigned long long u = __shfl_xor_sync(0xffffffffu, max_ulp, o);
    max_ulp = u > max_ulp ? u : max_ulp;
    const double m = __shfl_xor_sync(0xffffffffu, max_abs, o);
    max_abs = m > max_abs ? m : max_abs;
  }
  if ((threadIdx.x & 31) == 0) {
    if (n_diff) atomicAdd(&out[0], n_diff);
    if (zero) atomicAdd(&out[1], zero);
    if (nan_one) atomicAdd(&out[2], nan_one);
    if (measured) atomicAdd(&out[3], measured);
    atomicMax(&out[4], max_ulp);
    atomicMax(&out[5], (unsigned long long)__double_as_longlong(max_abs));   // non-negative doubles order as integers
  }
}

// bits[i / 32] bit (i % 32) set when 64-byte block i differs. `bytes` need not be a multiple of 64.
extern "C" __global__ void __launch_bounds__(256)
    kern_changed_blocks(const uint8_t* pre, const uint8_t* post, unsigned long long bytes, unsigned* bits) {
  const unsigned long long blocks = (bytes + 63) / 64;
  for (unsigned long long i = blockIdx.x * 256ull + threadIdx.x; i < blocks; i += (unsigned long long)gridDim.x * 256ull) {
    const unsigned long long lo = i * 64, hi = lo + 64 < bytes ? lo + 64 : bytes;
    bool diff = false;
    if (hi - lo == 64 && (reinterpret_cast<uintptr_t>(pre) % 16) == 0 && (reinterpret_cast<uintptr_t>(post) % 16) == 0) {
      for (int v = 0; v < 4; ++v) {
        const uint4 x = reinterpret_cast<const uint4*>(pre + lo)[v], y = reinterpret_cast<const uint4*>(post + lo)[v];
        diff |= (x.x != y.x) | (x.y != y.y) | (x.z != y.z) | (x.w != y.w);
      }
    } else {
      for (unsigned long long j = lo; j < hi; ++j) diff |= pre[j] != post[j];
    }
    if (diff) atomicOr(&bits[i / 32], 1u << (i % 32));
  }
}

// grid rows, block 256. out[row] = {argmax_a, argmax_b, top-1 margin of A (f32 bits), KL(A || B) (f32 bits)}.
extern "C" __global__ void __launch_bounds__(256)
    kern_logit_rows(const uint8_t* a, const uint8_t* b, unsigned cols, int dtype, unsigned long long stride_elems,
                    unsigned long long* out) {
  __shared__ float sv[8][4];
  __shared__ int si[8][2];
  const size_t base = (size_t)blockIdx.x * stride_elems;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float ma = -INFINITY, ma2 = -INFINITY, mb = -INFINITY;
  int ia = 0x7fffffff, ib = 0x7fffffff;
  long long dummy;
  for (unsigned c = threadIdx.x; c < cols; c += 256) {
    const float x = load_as_f32(a, base + c, dtype, dummy), y = load_as_f32(b, base + c, dtype, dummy);
    if (x > ma) { ma2 = ma; ma = x; ia = c; } else if (x > ma2) ma2 = x;
    if (y > mb) { mb = y; ib = c; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float oa = __shfl_xor_sync(0xffffffffu, ma, o), oa2 = __shfl_xor_sync(0xffffffffu, ma2, o);
    const int oia = __shfl_xor_sync(0xffffffffu, ia, o);
    if (oa > ma || (oa == ma && oia < ia)) { ma2 = fmaxf(ma, oa2); ma = oa; ia = oia; } else ma2 = fmaxf(ma2, oa);
    const float ob = __shfl_xor_sync(0xffffffffu, mb, o);
    const int oib = __shfl_xor_sync(0xffffffffu, ib, o);
    if (ob > mb || (ob == mb && oib < ib)) { mb = ob; ib = oib; }
  }
  if (lane == 0) { sv[warp][0] = ma; sv[warp][1] = ma2; sv[warp][2] = mb; si[warp][0] = ia; si[warp][1] = ib; }
  __syncthreads();
  ma = sv[0][0]; ma2 = sv[0][1]; mb = sv[0][2]; ia = si[0][0]; ib = si[0][1];
  for (int w = 1; w < 8; ++w) {
    if (sv[w][0] > ma || (sv[w][0] == ma && si[w][0] < ia)) { ma2 = fmaxf(ma, sv[w][1]); ma = sv[w][0]; ia = si[w][0]; }
    else ma2 = fmaxf(ma2, sv[w][0]);
    if (sv[w][2] > mb || (sv[w][2] == mb && si[w][1] < ib)) { mb = sv[w][2]; ib = si[w][1]; }
  }
  __syncthreads();
  // log-sum-exp of both rows, then KL(A || B) = sum pa (log pa - log pb)
  float za = 0.f, zb = 0.f;
  for (unsigned c = threadIdx.x; c < cols; c += 256) {
    za += __expf(load_as_f32(a, base + c, dtype, dummy) - ma);
    zb += __expf(load_as_f32(b, base + c, dtype, dummy) - mb);
  }
  za = warp_sum(za); zb = warp_sum(zb);
  if (lane == 0) { sv[warp][0] = za; sv[warp][1] = zb; }
  __syncthreads();
  za = 0.f; zb = 0.f;
  for (int w = 0; w < 8; ++w) { za += sv[w][0]; zb += sv[w][1]; }
  const float la = ma + __logf(za), lb = mb + __logf(zb);
  float kl = 0.f;
  for (unsigned c = threadIdx.x; c < cols; c += 256) {
    const float x = load_as_f32(a, base + c, dtype, dummy) - la, y = load_as_f32(b, base + c, dtype, dummy) - lb;
    kl += __expf(x) * (x - y);
  }
  kl = warp_sum(kl);
  __syncthreads();
  if (lane == 0) sv[warp][2] = kl;
  __syncthreads();
  if (threadIdx.x == 0) {
    kl = 0.f;
    for (int w = 0; w < 8; ++w) kl += sv[w][2];
    unsigned long long* o = out + (size_t)blockIdx.x * 4;
    o[0] = (unsigned long long)ia; o[1] = (unsigned long long)ib;
    o[2] = __float_as_uint(ma - ma2); o[3] = __float_as_uint(kl);
  }
}
