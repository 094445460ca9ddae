// Row-wise bandwidth-bound ops of the decoder: embedding gather, RMSNorm (plain, fused residual
// add, "weight + 1" Gemma form), SwiGLU / sigmoid gating as standalone ops for manifests that do
// not fuse them into a GEMM epilogue.
// Reference counterparts: tools/kernels-src/embedding.cu:6, gemma_rms_norm.cu:180,202,
// silu_mul.cu:10, sigmoid_mul.cu:14. These versions move 16 bytes per thread per access, keep the
// row in registers between the two passes of the norm, and take explicit extents.
#include "common.cuh"

namespace kern {

template <typename IdT>
KERN_DEVICE void embedding_body(const IdT* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                __nv_bfloat16* __restrict__ out, int tokens, int hidden, int vocab,
                                int* err) {
  const int t = blockIdx.x;
  if (t >= tokens) return;
  long long id = (long long)ids[t];
  if (id < 0 || id >= vocab) {
    set_error(err, ERR_BOUNDS);
    id = 0;
  }
  const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)id * hidden);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)t * hidden);
  if (!KERN_CHECK(src, (size_t)hidden * 2, SITE_EMBED_ROW)) return;
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dst[i] = src[i];
}

// y = x * rsqrt(mean(x^2) + eps) * (w [+ 1]); optional residual: r += x first, y = norm(r).
// One row per CTA; each thread keeps up to MAXV 16-byte vectors of the row in registers.
template <int MAXV, bool ADD>
KERN_DEVICE void rmsnorm_body(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* residual,
                              const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                              int rows, int n, int x_stride, int y_stride, float eps, int plus_one) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  if (row >= rows) return;
  const int nv = n / 8;
  const uint4* xv = reinterpret_cast<const uint4*>(x + (size_t)row * x_stride);
  uint4* rv = ADD ? reinterpret_cast<uint4*>(residual + (size_t)row * n) : nullptr;
  float vals[MAXV][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    if (i < nv) {
      uint4 u = xv[i];
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z),
             d = unpack_bf16x2(u.w);
      float v[8] = {a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y};
      if (ADD) {
        uint4 r = rv[i];
        float2 ra = unpack_bf16x2(r.x), rb = unpack_bf16x2(r.y), rc = unpack_bf16x2(r.z),
               rd = unpack_bf16x2(r.w);
        float rr[8] = {ra.x, ra.y, rb.x, rb.y, rc.x, rc.y, rd.x, rd.y};
        uint4 o;
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] += rr[e];
        o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
        o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
        rv[i] = o;
        // the norm reads the rounded residual, as a separate add kernel followed by a norm would
        float2 qa = unpack_bf16x2(o.x), qb = unpack_bf16x2(o.y), qc = unpack_bf16x2(o.z),
               qd = unpack_bf16x2(o.w);
        v[0] = qa.x; v[1] = qa.y; v[2] = qb.x; v[3] = qb.y;
        v[4] = qc.x; v[5] = qc.y; v[6] = qd.x; v[7] = qd.y;
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        vals[j][e] = v[e];
        ss += v[e] * v[e];
      }
    }
  }
  ss = warp_sum(ss);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  if (warp == 0) {
    float t = lane < (blockDim.x >> 5) ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[0] = t;
  }
  __syncthreads();
  const float inv = rsqrtf(red[0] / (float)n + eps);
  const uint4* wv = reinterpret_cast<const uint4*>(w);
  uint4* yv = reinterpret_cast<uint4*>(y + (size_t)row * y_stride);
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    if (i < nv) {
      uint4 u = wv[i];
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z),
             d = unpack_bf16x2(u.w);
      float ww[8] = {a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y};
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = vals[j][e] * inv * (plus_one ? ww[e] + 1.f : ww[e]);
      uint4 q;
      q.x = pack_bf16x2(o[0], o[1]); q.y = pack_bf16x2(o[2], o[3]);
      q.z = pack_bf16x2(o[4], o[5]); q.w = pack_bf16x2(o[6], o[7]);
      yv[i] = q;
    }
  }
}

}  // namespace kern

using namespace kern;

extern "C" __global__ void kern_embedding_i64_bf16(const long long* ids, const __nv_bfloat16* table,
                                                   __nv_bfloat16* out, int tokens, int hidden,
                                                   int vocab, int* err) {
  pdl_wait();
  embedding_body<long long>(ids, table, out, tokens, hidden, vocab, err);
}
extern "C" __global__ void kern_embedding_i32_bf16(const int* ids, const __nv_bfloat16* table,
                                                   __nv_bfloat16* out, int tokens, int hidden,
                                                   int vocab, int* err) {
  pdl_wait();
  embedding_body<int>(ids, table, out, tokens, hidden, vocab, err);
}

// block = 256 threads; n <= 256 * 8 * 4 = 8192 (the _wide entry covers up to 16384)
extern "C" __global__ void __launch_bounds__(256)
    kern_rms_norm_bf16(const __nv_bfloat16* x, const __nv_bfloat16* w, __nv_bfloat16* y, int rows,
                       int n, int x_stride, int y_stride, float eps, int plus_one) {
  pdl_wait();
  rmsnorm_body<4, false>(x, nullptr, w, y, rows, n, x_stride, y_stride, eps, plus_one);
  pdl_launch_dependents();
}
extern "C" __global__ void __launch_bounds__(256)
    kern_rms_norm_wide_bf16(const __nv_bfloat16* x, const __nv_bfloat16* w, __nv_bfloat16* y,
                            int rows, int n, int x_stride, int y_stride, float eps, int plus_one) {
  pdl_wait();
  rmsnorm_body<8, false>(x, nullptr, w, y, rows, n, x_stride, y_stride, eps, plus_one);
  pdl_launch_dependents();
}
// residual[row] += x[row]; y[row] = norm(residual[row])
extern "C" __global__ void __launch_bounds__(256)
    kern_fused_add_rms_norm_bf16(const __nv_bfloat16* x, __nv_bfloat16* residual,
                                 const __nv_bfloat16* w, __nv_bfloat16* y, int rows, int n,
                                 float eps, int plus_one) {
  pdl_wait();
  rmsnorm_body<8, true>(x, residual, w, y, rows, n, n, n, eps, plus_one);
  pdl_launch_dependents();
}

// out[t, j] = silu(x[t, j]) * x[t, d + j]      (x row = [gate | up], 2d wide)
extern "C" __global__ void kern_silu_mul_bf16(const __nv_bfloat16* x, __nv_bfloat16* out, int tokens,
                                              int d) {
  pdl_wait();
  const int t = blockIdx.x;
  if (t >= tokens) return;
  const uint4* g = reinterpret_cast<const uint4*>(x + (size_t)t * 2 * d);
  const uint4* u = reinterpret_cast<const uint4*>(x + (size_t)t * 2 * d + d);
  uint4* o = reinterpret_cast<uint4*>(out + (size_t)t * d);
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < d / 8; i += gridDim.y * blockDim.x) {
    uint4 a = g[i], b = u[i], r;
    float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z),
           a3 = unpack_bf16x2(a.w);
    float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y), b2 = unpack_bf16x2(b.z),
           b3 = unpack_bf16x2(b.w);
    r.x = pack_bf16x2(silu(a0.x) * b0.x, silu(a0.y) * b0.y);
    r.y = pack_bf16x2(silu(a1.x) * b1.x, silu(a1.y) * b1.y);
    r.z = pack_bf16x2(silu(a2.x) * b2.x, silu(a2.y) * b2.y);
    r.w = pack_bf16x2(silu(a3.x) * b3.x, silu(a3.y) * b3.y);
    o[i] = r;
  }
}

// out[t, j] = x[t, j] * sigmoid(gate[t, j])     (attention output gate)
extern "C" __global__ void kern_sigmoid_mul_bf16(const __nv_bfloat16* x, const __nv_bfloat16* gate,
                                                 __nv_bfloat16* out, int tokens, int d, int x_stride,
                                                 int gate_stride) {
  pdl_wait();
  const int t = blockIdx.x;
  if (t >= tokens) return;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < d; i += gridDim.y * blockDim.x) {
    float xv = __bfloat162float(x[(size_t)t * x_stride + i]);
    float gv = __bfloat162float(gate[(size_t)t * gate_stride + i]);
    out[(size_t)t * d + i] = __float2bfloat16(xv / (1.f + __expf(-gv)));
  }
}
