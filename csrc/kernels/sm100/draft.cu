// Helpers of speculative decoding with a block-draft model and of the recurrent state's advance after a round.
//
//   kern_topk_bf16          top-k (k <= 16) of every row of bf16 logits: ids (i64) and values (f32), larger value first,
//                           ties to the smaller index                      (reference: tools/kernels-src/topk_row.cu:21)
//   kern_mask_row0_bf16     copy rows, row 0 of every group of `rows_per_seq` set to -inf: on the gate inputs of the
//                           delta rule that makes the anchor's update the identity (decay 1, beta 0)
//                                                                          (reference: tools/kernels-src/gdn_advance.cu:26)
//   kern_conv_shift         move conv-window tokens a .. a+2 of a state line to 0 .. 2, a = accepted - 1
//                                                                          (reference: tools/kernels-src/gdn_advance.cu:36)
//   kern_dflash_conv_bf16   two-tap grouped conv of the block-draft model, in place; blocks of 8 tokens are independent
//                           (the second tap is masked at a block's first token), so the grid is (block, channel)
//                                                                          (reference: tools/kernels-src/dflash_conv.cu:19)
//   kern_dflash_select      greedy walk over `steps` draft positions with 16 candidates each: rank-R bilinear edge
//                           score between the previous choice and each candidate  (reference: tools/kernels-src/dflash_select.cu:26)
#include "common.cuh"

using namespace kern;

namespace {
constexpr int TOPK_MAX = 16;
KERN_DEVICE bool better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }
KERN_DEVICE float bf16r(float x) { return __bfloat162float(__float2bfloat16(x)); }
}  // namespace

// grid = rows, block 256. A thread keeps the best k of its strided slice (insertion into a sorted register list);
// then k rounds: every thread offers the head of its list, the block takes the best offer (shuffles inside a warp,
// one shared-memory hop across the 8 warps) and its owner moves on.
extern "C" __global__ void __launch_bounds__(256)
    kern_topk_bf16(const __nv_bfloat16* logits, long long* ids, float* vals, int n, int row_stride, int k) {
  pdl_wait();
  __shared__ float wv[8];
  __shared__ int wi[8];
  const __nv_bfloat16* row = logits + (size_t)blockIdx.x * row_stride;
  k = min(k, TOPK_MAX);
  float lv[TOPK_MAX];
  int li[TOPK_MAX];
#pragma unroll
  for (int j = 0; j < TOPK_MAX; ++j) { lv[j] = -INFINITY; li[j] = 0x7fffffff; }
  for (int i = threadIdx.x; i < n; i += 256) {
    const float v = __bfloat162float(row[i]);
    if (!better(v, i, lv[TOPK_MAX - 1], li[TOPK_MAX - 1])) continue;
    // bubble the newcomer up from the tail (static indices keep the list in registers)
    lv[TOPK_MAX - 1] = v;
    li[TOPK_MAX - 1] = i;
#pragma unroll
    for (int j = TOPK_MAX - 1; j > 0; --j) {
      if (better(lv[j], li[j], lv[j - 1], li[j - 1])) {
        const float tv = lv[j]; lv[j] = lv[j - 1]; lv[j - 1] = tv;
        const int ti = li[j]; li[j] = li[j - 1]; li[j - 1] = ti;
      }
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int r = 0; r < k; ++r) {
    float bv = lv[0];
    int bi = li[0];
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { wv[warp] = bv; wi[warp] = bi; }
    __syncthreads();
    float gv = wv[0];
    int gi = wi[0];
#pragma unroll
    for (int w = 1; w < 8; ++w)
      if (better(wv[w], wi[w], gv, gi)) { gv = wv[w]; gi = wi[w]; }
    if (li[0] == gi && gi != 0x7fffffff) {      // indices are unique: exactly one thread owns the winner
#pragma unroll
      for (int j = 0; j < TOPK_MAX - 1; ++j) { lv[j] = lv[j + 1]; li[j] = li[j + 1]; }
      lv[TOPK_MAX - 1] = -INFINITY;
      li[TOPK_MAX - 1] = 0x7fffffff;
    }
    if (threadIdx.x == 0) {
      ids[(size_t)blockIdx.x * k + r] = gi == 0x7fffffff ? -1 : gi;
      vals[(size_t)blockIdx.x * k + r] = gv;
    }
    __syncthreads();
  }
}

// grid = rows, block 128.
extern "C" __global__ void __launch_bounds__(128)
    kern_mask_row0_bf16(__nv_bfloat16* dst, const __nv_bfloat16* src, int rows, int rows_per_seq, int cols) {
  pdl_wait();
  const int r = blockIdx.x;
  if (r >= rows) return;
  const bool masked = (r % rows_per_seq) == 0;
  const __nv_bfloat16 ninf = __float2bfloat16(-INFINITY);
  for (int c = threadIdx.x; c < cols; c += 128) dst[(size_t)r * cols + c] = masked ? ninf : src[(size_t)r * cols + c];
}

// grid [seqs, ceil(tok_bytes / 16 / 128)], block 128. The line of sequence s is lines[s * line_stride + a]; a thread
// reads its three 16-byte vectors before it writes any (the ranges overlap when a < 3). Line 0 and a <= 0 are no-ops.
extern "C" __global__ void __launch_bounds__(128)
    kern_conv_shift(const int* lines, int line_stride, uint8_t* state, const int* accepted, int seqs, long long line_bytes,
                    long long tok_bytes) {
  pdl_wait();
  const int s = blockIdx.x;
  if (s >= seqs) return;
  const long long a = (long long)accepted[s] - 1;
  if (a <= 0) return;
  const long long line = lines[(size_t)s * line_stride + a];
  if (line <= 0) return;
  const long long v = (long long)blockIdx.y * 128 + threadIdx.x;
  if (v * 16 >= tok_bytes) return;
  uint8_t* base = state + line * line_bytes + v * 16;
  const uint4 t0 = *reinterpret_cast<const uint4*>(base + a * tok_bytes);
  const uint4 t1 = *reinterpret_cast<const uint4*>(base + (a + 1) * tok_bytes);
  const uint4 t2 = *reinterpret_cast<const uint4*>(base + (a + 2) * tok_bytes);
  *reinterpret_cast<uint4*>(base) = t0;
  *reinterpret_cast<uint4*>(base + tok_bytes) = t1;
  *reinterpret_cast<uint4*>(base + 2 * tok_bytes) = t2;
}

// coef[t, tap, ch] = base[side, tap, ch] + delta[t, side, tap, group(ch)];
// out[t, ch] = coef[t, 0, ch] x[t, ch] + coef[t, 1, ch] x[t-1, ch] (t % 8 != 0); every intermediate rounded to bf16.
// grid [ceil(tokens / 8), ceil(dim / 256)], block 256: a thread walks the 8 tokens of its block for one channel.
extern "C" __global__ void __launch_bounds__(256)
    kern_dflash_conv_bf16(__nv_bfloat16* x, const __nv_bfloat16* delta, const __nv_bfloat16* base, int tokens, int dim,
                          int groups, int delta_stride, int side) {
  pdl_wait();
  const int ch = blockIdx.y * 256 + threadIdx.x;
  const int t0 = blockIdx.x * 8;
  if (ch >= dim || t0 >= tokens) return;
  const int g = ch / (dim / groups);
  const float b0 = __bfloat162float(base[(size_t)(side * 2 + 0) * dim + ch]);
  const float b1 = __bfloat162float(base[(size_t)(side * 2 + 1) * dim + ch]);
  float prev = 0.f;
  for (int t = t0; t < min(tokens, t0 + 8); ++t) {
    const float xt = __bfloat162float(x[(size_t)t * dim + ch]);
    const __nv_bfloat16* dl = delta + (size_t)t * delta_stride + side * 2 * groups;
    const float c0 = bf16r(b0 + __bfloat162float(dl[g]));
    const float c1 = bf16r(b1 + __bfloat162float(dl[groups + g]));
    const float a0 = bf16r(c0 * xt);
    const float a1 = t == t0 ? 0.f : bf16r(c1 * prev);
    x[(size_t)t * dim + ch] = __float2bfloat16(a0 + a1);
    prev = xt;
  }
}

// grid = seqs, block = rank (a multiple of 32, at most 1024). Rows of sequence s are rows_per_seq consecutive rows of
// cand / unary / hidden_r / succ / pred, row 0 the anchor; step l reads row s * rows_per_seq + 1 + l.
//   s[c] = unary[row, c] + bf16( sum_r bf16(pred_row[r] * hidden_r[row, r]) * succ[row, c, r] ),  pick the first maximum
extern "C" __global__ void __launch_bounds__(1024)
    kern_dflash_select(const long long* cand, const float* unary, const __nv_bfloat16* hidden_r, const __nv_bfloat16* succ,
                       const __nv_bfloat16* pred, const __nv_bfloat16* pred_anchor, long long* out, int steps, int rank,
                       int hr_stride, int rows_per_seq) {
  pdl_wait();
  constexpr int KC = 16;
  __shared__ float part[32][KC];
  __shared__ int prev_s;
  const int r = threadIdx.x, warp = r >> 5, lane = r & 31, warps = (rank + 31) >> 5;
  const long long seq = blockIdx.x, row0 = seq * rows_per_seq + 1;
  int prev = 0;
  for (int l = 0; l < steps; ++l) {
    const long long row = row0 + l;
    const __nv_bfloat16* pr = l == 0 ? pred_anchor + seq * rank : pred + ((row - 1) * KC + prev) * rank;
    const float ph = r < rank ? bf16r(__bfloat162float(pr[r]) * __bfloat162float(hidden_r[row * hr_stride + r])) : 0.f;
#pragma unroll
    for (int c = 0; c < KC; ++c) {
      const float v = r < rank ? ph * __bfloat162float(succ[(row * KC + c) * rank + r]) : 0.f;
      const float s = warp_sum(v);
      if (lane == 0) part[warp][c] = s;
    }
    __syncthreads();
    if (r == 0) {
      int best = 0;
      float bs = -INFINITY;
      for (int c = 0; c < KC; ++c) {
        float s = 0.f;
        for (int w = 0; w < warps; ++w) s += part[w][c];
        s = unary[row * KC + c] + bf16r(s);
        if (s > bs) { bs = s; best = c; }
      }
      out[seq * steps + l] = cand[row * KC + best];
      prev_s = best;
    }
    __syncthreads();
    prev = prev_s;
  }
}
