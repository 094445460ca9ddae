// Attention preparation in one pass over a token's fused QKV row: optional per-head RMSNorm of q
// and k (QK-norm, plain or "weight + 1"), rotary embedding over the first `rot` dims of each head
// (rotate-half pairing) from an f32 cos/sin table, q rewritten in place, k and v appended to the
// paged KV cache at the token's slot.
// Reference counterpart: tools/kernels-src/attn_prep.cu:152 (fixed QH 24 / KH 4 / HD 256 / RD 64);
// this version takes head counts, head dim, rotary dim and page size as arguments.
//
// KV cache layout of one layer: [page][k|v][kv_head][page_size][head_dim] bf16, so one
// (page, k|v, head) block is one contiguous page_size x head_dim tile that a 2-D TMA box or a
// 1-D bulk copy fetches whole. slot = page * page_size + offset; slot < 0 skips the append.
#include "common.cuh"

using namespace kern;

// grid = tokens, block = 128 (4 warps, heads dealt to warps), dyn smem = 4 * head_dim * 4 bytes
extern "C" __global__ void __launch_bounds__(128)
    kern_rope_kv_append_bf16(__nv_bfloat16* qkv, __nv_bfloat16* kv, const long long* positions,
                             const long long* slots, const float* cos_tab, const float* sin_tab,
                             const __nv_bfloat16* q_norm, const __nv_bfloat16* k_norm, int tokens,
                             int hq, int hk, int d, int rot, int page_size, float eps,
                             int norm_plus_one, long long kv_slots, int max_pos, int row_stride, int* err) {
  extern __shared__ float rows[];  // [4][d]
  pdl_wait();
  const int t = blockIdx.x;
  if (t >= tokens) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* row = rows + warp * d;
  long long pos = positions[t];
  long long slot = slots[t];
  if (pos < 0 || pos >= max_pos) {
    set_error(err, ERR_BOUNDS);
    pos = 0;
  }
  if (slot >= kv_slots) {
    set_error(err, ERR_BOUNDS);
    slot = -1;
  }
  const int half = rot >> 1;
  const float* cs = cos_tab + (size_t)pos * half;
  const float* sn = sin_tab + (size_t)pos * half;
  __nv_bfloat16* base = qkv + (size_t)t * row_stride;   // a row may carry more than q|k|v (an output gate)
  const long long page = slot >= 0 ? slot / page_size : 0;
  const int off = slot >= 0 ? (int)(slot % page_size) : 0;
  const size_t page_elems = (size_t)2 * hk * page_size * d;

  for (int h = warp; h < hq + 2 * hk; h += 4) {
    __nv_bfloat16* src = base + (size_t)h * d;
    const bool is_q = h < hq, is_k = !is_q && h < hq + hk;
    if (!is_q && slot < 0) continue;
    __nv_bfloat16* dst;
    if (is_q) {
      dst = src;
    } else {
      const int kvh = is_k ? h - hq : h - hq - hk;
      dst = kv + (size_t)page * page_elems + ((size_t)(is_k ? 0 : 1) * hk + kvh) * page_size * d +
            (size_t)off * d;
      if (!KERN_CHECK(dst, (size_t)d * 2, SITE_KV_APPEND)) continue;
    }
    if (!is_q && !is_k) {  // v: straight copy
      for (int i = lane; i < d / 8; i += 32)
        reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
      continue;
    }
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) {
      float v = __bfloat162float(src[i]);
      row[i] = v;
      ss += v * v;
    }
    const __nv_bfloat16* nw = is_q ? q_norm : k_norm;
    float inv = 1.f;
    if (nw != nullptr) {
      ss = warp_sum(ss);
      inv = rsqrtf(ss / (float)d + eps);
    }
    __syncwarp();
    for (int i = lane; i < d; i += 32) {
      float v = row[i] * inv;
      if (nw != nullptr) {
        float w = __bfloat162float(nw[i]);
        v *= norm_plus_one ? w + 1.f : w;
        // the norm's output is rounded to bf16 before the rotation, as separate kernels would
        v = __bfloat162float(__float2bfloat16(v));
      }
      float o = v;
      if (i < rot) {
        const int j = i < half ? i : i - half;
        const int pi = i < half ? i + half : i - half;
        float pv = row[pi] * inv;
        if (nw != nullptr) {
          float w = __bfloat162float(nw[pi]);
          pv *= norm_plus_one ? w + 1.f : w;
          pv = __bfloat162float(__float2bfloat16(pv));
        }
        const float c = cs[j], s = sn[j];
        o = i < half ? v * c - pv * s : v * c + pv * s;
      }
      dst[i] = __float2bfloat16(o);
    }
    __syncwarp();
  }
  pdl_launch_dependents();
}

// cos/sin tables [max_pos][rot/2] in f32, angles evaluated in double so large positions stay exact.
extern "C" __global__ void kern_rope_table_f32(float* cos_tab, float* sin_tab, int max_pos, int rot,
                                               double theta) {
  const int half = rot >> 1;
  const long long n = (long long)max_pos * half;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const int j = (int)(i % half);
    const long long p = i / half;
    const double inv_freq = pow(theta, -2.0 * (double)j / (double)rot);
    double s, c;
    sincos((double)p * inv_freq, &s, &c);
    cos_tab[i] = (float)c;
    sin_tab[i] = (float)s;
  }
}
