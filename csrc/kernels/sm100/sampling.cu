// Token selection: greedy argmax (ties -> lowest index, two stages so one row uses many SMs), and
// temperature / top-k / top-p / min-p sampling over f32 or bf16 logits with a counter-based RNG whose
// draw depends only on (seed, row offset) so a replayed step repeats its choice.
// Reference counterparts: tools/kernels-src/argmax.cu:38,58 (partial + final),
// tools/kernels-src/sample_glue.cu:10,24,40 and the FlashInfer sampling instantiations named in
// kernel_index/flashinfer_sampling.toml (top-k / top-p renorm + min-p sampling). This file replaces
// that chain with one row-per-CTA kernel that sorts nothing: it finds the top-k / top-p / min-p
// thresholds by bisection on the probability value.
#include "common.cuh"

using namespace kern;

template <typename T>
KERN_DEVICE float to_f32(T v);
template <>
KERN_DEVICE float to_f32<float>(float v) { return v; }
template <>
KERN_DEVICE float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

KERN_DEVICE void argmax_combine(float& bv, int& bi, float v, int i) {
  if (v > bv || (v == bv && i < bi)) {
    bv = v;
    bi = i;
  }
}

template <typename T>
KERN_DEVICE void argmax_partial_body(const T* logits, float* pv, int* pi, int rows, int vocab,
                                     int stride) {
  __shared__ float sv[32];
  __shared__ int si[32];
  const int row = blockIdx.x, part = blockIdx.y, parts = gridDim.y;
  if (row >= rows) return;
  const int per = (vocab + parts - 1) / parts;
  const int lo = part * per, hi = min(vocab, lo + per);
  const T* x = logits + (size_t)row * stride;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    float v = to_f32<T>(x[i]);
    if (v != v) v = -INFINITY;  // a NaN never wins
    argmax_combine(bv, bi, v, i);
  }
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    argmax_combine(bv, bi, ov, oi);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    sv[warp] = bv;
    si[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    bv = lane < (blockDim.x >> 5) ? sv[lane] : -INFINITY;
    bi = lane < (blockDim.x >> 5) ? si[lane] : 0x7fffffff;
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      argmax_combine(bv, bi, ov, oi);
    }
    if (lane == 0) {
      pv[(size_t)row * parts + part] = bv;
      pi[(size_t)row * parts + part] = bi;
    }
  }
}

// grid [rows, parts], block 256
extern "C" __global__ void kern_argmax_partial_bf16(const __nv_bfloat16* logits, float* pv, int* pi,
                                                    int rows, int vocab, int stride) {
  pdl_wait();
  argmax_partial_body<__nv_bfloat16>(logits, pv, pi, rows, vocab, stride);
}
extern "C" __global__ void kern_argmax_partial_f32(const float* logits, float* pv, int* pi, int rows,
                                                   int vocab, int stride) {
  pdl_wait();
  argmax_partial_body<float>(logits, pv, pi, rows, vocab, stride);
}
// grid [rows], block 32
extern "C" __global__ void kern_argmax_final_i64(const float* pv, const int* pi, long long* out,
                                                 int rows, int parts) {
  pdl_wait();
  const int row = blockIdx.x;
  if (row >= rows) return;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int p = threadIdx.x; p < parts; p += 32)
    argmax_combine(bv, bi, pv[(size_t)row * parts + p], pi[(size_t)row * parts + p]);
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    argmax_combine(bv, bi, ov, oi);
  }
  if (threadIdx.x == 0) out[row] = bi == 0x7fffffff ? 0 : bi;
}

// ---- stochastic sampling ------------------------------------------------------------------------
// splitmix64 -> uniform in [0,1): the draw is a pure function of (seed, offset)
KERN_DEVICE float uniform01(unsigned long long seed, unsigned long long offset) {
  unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (offset + 1);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z = z ^ (z >> 31);
  return (float)(z >> 40) * (1.0f / 16777216.0f);
}

KERN_DEVICE float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < (blockDim.x >> 5) ? red[lane] : 0.f;
  t = warp_sum(t);
  return __shfl_sync(0xffffffffu, t, 0);
}
KERN_DEVICE float block_max(float v, float* red) {
  v = warp_max(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < (blockDim.x >> 5) ? red[lane] : -INFINITY;
  t = warp_max(t);
  return __shfl_sync(0xffffffffu, t, 0);
}

// One row per CTA (block 1024). probs scratch: f32 [rows, vocab]. temperature <= 0 -> greedy.
// Filters compose in the usual order: top-k, then top-p over the renormalised survivors, then min-p.
// The kept set is {p >= threshold}; the threshold comes from 24 bisection steps, then one inverse-CDF
// walk picks the token: lowest index whose running sum exceeds u * kept_mass.
template <typename T>
KERN_DEVICE void sample_body(const T* logits, float* probs, long long* out, const float* temperature,
                             const int* top_k, const float* top_p, const float* min_p,
                             const long long* seeds, const int* offsets, int rows, int vocab,
                             int stride) {
  __shared__ float red[32];
  __shared__ float scan[1024];
  const int row = blockIdx.x;
  if (row >= rows) return;
  const T* x = logits + (size_t)row * stride;
  float* p = probs + (size_t)row * vocab;
  const float temp = temperature ? temperature[row] : 0.f;
  // greedy rows reuse the argmax rule (ties -> lowest index)
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    float v = to_f32<T>(x[i]);
    if (v != v) v = -INFINITY;
    argmax_combine(bv, bi, v, i);
  }
  const float mx = block_max(bv, red);
  if (temp <= 0.f) {
    int cand = (bv == mx) ? bi : 0x7fffffff;
    for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    __shared__ int best[32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) best[warp] = cand;
    __syncthreads();
    if (threadIdx.x == 0) {
      int b = 0x7fffffff;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) b = min(b, best[w]);
      out[row] = b == 0x7fffffff ? 0 : b;
    }
    return;
  }
  const float inv_t = 1.f / temp;
  float s = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    float v = to_f32<T>(x[i]);
    float e = (v != v) ? 0.f : __expf((v - mx) * inv_t);
    p[i] = e;
    s += e;
  }
  const float total = block_sum(s, red);
  const float inv_total = 1.f / total;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) p[i] *= inv_total;
  __syncthreads();

  float thresh = 0.f;  // keep p >= thresh
  const int k = top_k ? top_k[row] : 0;
  if (k > 0 && k < vocab) {
    float lo = 0.f, hi = 1.f;  // count(p >= lo) >= k > count(p >= hi)  (hi exclusive bound)
    for (int it = 0; it < 24; ++it) {
      const float mid = 0.5f * (lo + hi);
      float c = 0.f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) c += p[i] >= mid ? 1.f : 0.f;
      c = block_sum(c, red);
      if (c >= (float)k) lo = mid; else hi = mid;
    }
    thresh = lo;
  }
  const float tp = top_p ? top_p[row] : 1.f;
  if (tp < 1.f) {
    float kept = 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) kept += p[i] >= thresh ? p[i] : 0.f;
    kept = block_sum(kept, red);
    // largest t with mass(p >= t) >= tp * kept
    float lo = thresh, hi = 1.f;
    for (int it = 0; it < 24; ++it) {
      const float mid = 0.5f * (lo + hi);
      float c = 0.f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) c += p[i] >= mid ? p[i] : 0.f;
      c = block_sum(c, red);
      if (c >= tp * kept) lo = mid; else hi = mid;
    }
    thresh = lo;
  }
  const float mp = min_p ? min_p[row] : 0.f;
  if (mp > 0.f) {
    const float pmax = inv_total;  // exp(0) / total
    thresh = fmaxf(thresh, mp * pmax);
  }
  float kept = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) kept += p[i] >= thresh ? p[i] : 0.f;
  kept = block_sum(kept, red);
  const unsigned long long seed = seeds ? (unsigned long long)seeds[row] : 0ull;
  const unsigned long long off = offsets ? (unsigned long long)offsets[row] : 0ull;
  const float target = uniform01(seed, off) * kept;

  // inverse CDF: contiguous chunk per thread, block scan of chunk sums, then a walk in one chunk
  const int per = (vocab + blockDim.x - 1) / blockDim.x;
  const int lo_i = threadIdx.x * per, hi_i = min(vocab, lo_i + per);
  float mine = 0.f;
  for (int i = lo_i; i < hi_i; ++i) mine += p[i] >= thresh ? p[i] : 0.f;
  scan[threadIdx.x] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    float run = 0.f;
    int chosen_t = -1;
    for (int t = 0; t < (int)blockDim.x; ++t) {
      if (scan[t] > 0.f && run + scan[t] > target) {
        chosen_t = t;
        break;
      }
      run += scan[t];
    }
    if (chosen_t < 0) {  // rounding left target at the very end: take the last kept chunk
      for (int t = blockDim.x - 1; t >= 0; --t)
        if (scan[t] > 0.f) {
          chosen_t = t;
          run -= scan[t];
          break;
        }
    }
    int pick = bi == 0x7fffffff ? 0 : bi;
    if (chosen_t >= 0) {
      const int a = chosen_t * per, b = min(vocab, a + per);
      int last = -1;
      for (int i = a; i < b; ++i) {
        if (p[i] >= thresh) {
          last = i;
          run += p[i];
          if (run > target) break;
        }
      }
      if (last >= 0) pick = last;
    }
    out[row] = pick;
  }
}

extern "C" __global__ void __launch_bounds__(1024)
    kern_sample_f32(const float* logits, float* probs, long long* out, const float* temperature,
                    const int* top_k, const float* top_p, const float* min_p, const long long* seeds,
                    const int* offsets, int rows, int vocab, int stride) {
  pdl_wait();
  sample_body<float>(logits, probs, out, temperature, top_k, top_p, min_p, seeds, offsets, rows,
                     vocab, stride);
}
extern "C" __global__ void __launch_bounds__(1024)
    kern_sample_bf16(const __nv_bfloat16* logits, float* probs, long long* out,
                     const float* temperature, const int* top_k, const float* top_p,
                     const float* min_p, const long long* seeds, const int* offsets, int rows,
                     int vocab, int stride) {
  pdl_wait();
  sample_body<__nv_bfloat16>(logits, probs, out, temperature, top_k, top_p, min_p, seeds, offsets,
                             rows, vocab, stride);
}
