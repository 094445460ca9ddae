// Decode attention of multi-head latent attention in its absorbed form: every head attends over ONE shared latent
// cache, keys are the 576-wide latent rows (512 compressed + 64 rotary), values are the first 512 columns of the same
// rows — so a KV tile is fetched once and serves both products.
//
//   q      [seqs, H, 576] bf16 (q_nope absorbed through W_UK, then the rotary part)
//   cache  paged latent rows [page][page_size][576] bf16, one "kv head"
//   out    [seqs, H, 512] bf16 (the caller applies W_UV / o_proj), or split partials (o, m, l) for the usual merge
//
// A CTA owns 16 heads of one sequence (one m16 tile) and one KV split. MW math warps, a tile of 8 MW tokens: for
// S = Q K^T each warp takes 8 of the tile's tokens; the probabilities go through shared memory (all warps use the tile's
// common row maximum), and for O += P V each warp owns 512 / MW of the value columns — a warp's accumulator is
// 16 x 64, not 16 x 512. One more warp feeds the ring of tiles by TMA (nine 64-column boxes per tile, 128-byte
// swizzle). Tiles of 64 tokens (72 KB) in a two-stage ring, all eight warps score. Measured alternatives, both slower
// than this (0.167 ms for 64 sequences of 8192 rows): 48-token tiles three deep with six scoring warps (0.196 ms) and
// 32-token tiles four deep with four warps (0.203 ms) — more barriers and row-maximum exchanges per token cost more
// than the deeper ring gains.
// With 16 heads per rank (tensor parallel 8) a tile is read once per sequence; with more heads the CTAs of a sequence
// share the tile through L2. One row per sequence (decode); verify rows of a speculative round are not handled here.
// Reference: the reference takes this kernel from a CuTe-DSL build (MLA decode, sm100) and the context form from a
// prebuilt blob (kernel_index/trtllm_fmha_ctx_h192_v128.toml); neither has source there.
#include "common.cuh"

using namespace kern;

namespace {

constexpr int MW = 8;                    // math warps: 512 / MW value columns each for O
constexpr int TKM = 64;                  // tokens per tile
constexpr int SW = TKM / 8;              // warps that take part in S = Q K^T, 8 tokens of the tile each
constexpr int DQK = 576, DVV = 512;
constexpr int HM = 16;                   // heads per CTA
constexpr int kTileBytes = TKM * DQK * 2;
constexpr int kStagesM = TKM == 48 ? 3 : 2;   // 48-token tiles (54 KB) three deep, or 64-token tiles two deep
constexpr int ON = DVV / MW / 8;             // 8-column accumulator tiles per warp
constexpr int kQStride = DQK + 8, kPStride = TKM + 8;
constexpr int kQBytes = HM * kQStride * 2, kPBytes = HM * kPStride * 2;

KERN_DEVICE void ldsm4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
KERN_DEVICE void ldsm4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
KERN_DEVICE void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// byte offset of (token row, 16-byte chunk 0..71) in a tile stored as nine column blocks of [64 rows][128 bytes]
KERN_DEVICE uint32_t lat_off(int tok, int chunk) {
  const int cb = chunk >> 3, c = chunk & 7;
  return (uint32_t)(cb * (TKM * 128) + tok * 128 + ((c ^ (tok & 7)) << 4));
}
KERN_DEVICE void math_bar() { asm volatile("bar.sync 1, %0;" ::"n"(MW * 32) : "memory"); }

}  // namespace

// grid [ceil(H / 16), seqs, splits], block 32 MW + 32, dynamic shared memory MLA_SMEM bytes.
// `splits` packs (launch splits | first slot << 8 | slots per (row, head) << 16) as the GQA decode kernel does.
constexpr int MLA_SMEM = 1024 + kStagesM * kTileBytes + kQBytes + kPBytes + 2 * MW * HM * 4 + 128;

extern "C" __global__ void __launch_bounds__(MW * 32 + 32, 1)
    kern_mla_decode_bf16(const __grid_constant__ CUtensorMap lat_map, const __nv_bfloat16* q, __nv_bfloat16* out, float* ws_o,
                         float* ws_ml, const int* block_table, const int* seq_lens, int seqs, int heads, int q_stride,
                         int out_stride, int max_pages, int page_size, int splits, int pool_pages, float scale_log2, int* err,
                         const int* row_seq) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stages = smem;
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem + kStagesM * kTileBytes);
  __nv_bfloat16* ps = reinterpret_cast<__nv_bfloat16*>(smem + kStagesM * kTileBytes + kQBytes);
  float* sm_m = reinterpret_cast<float*>(smem + kStagesM * kTileBytes + kQBytes + kPBytes);      // [MW][16] tile maxima per warp
  float* sm_l = sm_m + MW * HM;                                                                  // [MW][16] row sums per warp
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sm_l + MW * HM);
  uint64_t* empty_bar = full_bar + kStagesM;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + kStagesM);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = blockIdx.y, head0 = blockIdx.x * HM, split = blockIdx.z;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStagesM; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], MW);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&lat_map);
  }
  __syncthreads();
  pdl_wait();
  if (seq >= seqs) return;
  const int L = seq_lens[seq];
  const int trow = row_seq != nullptr ? row_seq[seq] : seq;      // the block-table row: prefill rows share their sequence's
  const int valid_rows = min(HM, heads - head0);
  const int nsplit = splits & 0xff, split_base = (splits >> 8) & 0xff;
  const int split_total = (splits >> 16) ? (splits >> 16) : nsplit;
  if (L <= 0 || valid_rows <= 0) return;       // uniform per CTA
  const int ntiles_all = (L + TKM - 1) / TKM;
  int tile_lo = 0, tile_hi = ntiles_all;
  if (nsplit > 1) {
    const int per = (ntiles_all + nsplit - 1) / nsplit;
    tile_lo = split * per;
    tile_hi = min(ntiles_all, tile_lo + per);
    if (tile_hi < tile_lo) tile_hi = tile_lo;
  }
  const int ntiles = tile_hi - tile_lo;

  // the 16 query rows (one per head) -> shared
  for (int i = threadIdx.x; i < HM * (DQK / 8); i += blockDim.x) {
    const int r = i / (DQK / 8), c = i % (DQK / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < valid_rows) v = *reinterpret_cast<const uint4*>(q + (size_t)seq * q_stride + (size_t)(head0 + r) * DQK + c * 8);
    *reinterpret_cast<uint4*>(qs + r * kQStride + c * 8) = v;
  }
  __syncthreads();

  if (warp == MW) {
    // ---------------- producer ----------------
    if (lane == 0) {
      // a box never crosses a page: 16-row boxes for the 48-token tile, whole tiles (or pages) otherwise
      const int box_rows = TKM % 32 != 0 ? 16 : (page_size < TKM ? page_size : TKM);
      const int boxes = TKM / box_rows;
      int stage = 0;
      uint32_t phase = 0;
      for (int t = 0; t < ntiles; ++t) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
          set_error(err, ERR_WAIT_EMPTY);
          *abort_flag = 1;
          break;
        }
        uint8_t* sk = stages + stage * kTileBytes;
        mbar_expect_tx(&full_bar[stage], kTileBytes);
        const int tok0 = (tile_lo + t) * TKM;
        for (int b = 0; b < boxes; ++b) {
          const int tok = tok0 + b * box_rows;
          int page = 0, in_page = 0;
          const int pidx = tok / page_size;
          if (tok < L && pidx < max_pages) {
            page = block_table[(size_t)trow * max_pages + pidx];
            in_page = tok % page_size;
          }
          if (page < 0 || page >= pool_pages) {
            set_error(err, ERR_BOUNDS);
            page = 0;
          }
          const int row = page * page_size + in_page;
#pragma unroll
          for (int cb = 0; cb < DQK / 64; ++cb)
            tma_load_2d(sk + cb * (TKM * 128) + b * box_rows * 128, &lat_map, cb * 64, row, &full_bar[stage]);
        }
        if (++stage == kStagesM) { stage = 0; phase ^= 1; }
      }
    }
  }

  float o[ON][4];                       // this warp's 16 heads x (512 / MW) value columns
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
#pragma unroll
  for (int i = 0; i < ON; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  if (warp < MW) {
    const int rA = lane >> 2, rB = rA + 8;
    const uint32_t q_addr = smem_u32(qs) + (((lane & 7) + ((lane >> 3) & 1) * 8) * kQStride + (lane >> 4) * 8) * 2;
    const uint32_t p_addr = smem_u32(ps) + (((lane & 7) + ((lane >> 3) & 1) * 8) * kPStride + (lane >> 4) * 8) * 2;
    const int wtok = warp * 8;          // this warp's tokens inside a tile (for S)
    int stage = 0;
    uint32_t phase = 0;
    bool live = true;
    for (int t = 0; t < ntiles; ++t) {
      if (live && !mbar_wait(&full_bar[stage], phase, abort_flag)) {
        set_error(err, ERR_WAIT_FULL);
        *abort_flag = 1;
        live = false;
      }
      // the four warps meet at two barriers per tile, so a warp that gave up keeps walking (without touching the ring)
      const uint32_t sk = smem_u32(stages + stage * kTileBytes);
      const int tok0 = (tile_lo + t) * TKM;
      float s[1][4];
      s[0][0] = s[0][1] = s[0][2] = s[0][3] = 0.f;
      const bool scoring = live && warp < SW;
      if (scoring) {
#pragma unroll 2
        for (int kk = 0; kk < DQK / 16; kk += 2) {
          uint32_t qa[2][4];
          ldsm4(q_addr + kk * 32, qa[0][0], qa[0][1], qa[0][2], qa[0][3]);
          ldsm4(q_addr + kk * 32 + 32, qa[1][0], qa[1][1], qa[1][2], qa[1][3]);
#pragma unroll
          for (int n = 0; n < 1; ++n) {
            const int tok = wtok + n * 8 + (lane & 7);
            uint32_t b0, b1, b2, b3;
            ldsm4(sk + lat_off(tok, kk * 2 + (lane >> 3)), b0, b1, b2, b3);
            mma16816(s[n], qa[0][0], qa[0][1], qa[0][2], qa[0][3], b0, b1);
            mma16816(s[n], qa[1][0], qa[1][1], qa[1][2], qa[1][3], b2, b3);
          }
        }
      }
      float mxA = -INFINITY, mxB = -INFINITY;
#pragma unroll
      for (int n = 0; n < 1; ++n) {
        const int j = tok0 + wtok + n * 8 + 2 * (lane & 3);
        s[n][0] = (scoring && j < L) ? s[n][0] * scale_log2 : -INFINITY;
        s[n][1] = (scoring && j + 1 < L) ? s[n][1] * scale_log2 : -INFINITY;
        s[n][2] = (scoring && j < L) ? s[n][2] * scale_log2 : -INFINITY;
        s[n][3] = (scoring && j + 1 < L) ? s[n][3] * scale_log2 : -INFINITY;
        mxA = fmaxf(mxA, fmaxf(s[n][0], s[n][1]));
        mxB = fmaxf(mxB, fmaxf(s[n][2], s[n][3]));
      }
      mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1));
      mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
      mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1));
      mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
      if (warp < SW && (lane & 3) == 0) { sm_m[warp * HM + rA] = mxA; sm_m[warp * HM + rB] = mxB; }
      math_bar();                       // every scoring warp's tile maxima are in
      float tA = -INFINITY, tB = -INFINITY;
#pragma unroll
      for (int w = 0; w < SW; ++w) { tA = fmaxf(tA, sm_m[w * HM + rA]); tB = fmaxf(tB, sm_m[w * HM + rB]); }
      const float mA = fmaxf(m_run[0], tA), mB = fmaxf(m_run[1], tB);
      const float mA_use = mA == -INFINITY ? 0.f : mA, mB_use = mB == -INFINITY ? 0.f : mB;
      const float cA = exp2f(m_run[0] - mA_use), cB = exp2f(m_run[1] - mB_use);
      m_run[0] = mA;
      m_run[1] = mB;
      float sumA = 0.f, sumB = 0.f;
#pragma unroll
      for (int n = 0; n < 1; ++n) {
        const float p0 = exp2f(s[n][0] - mA_use), p1 = exp2f(s[n][1] - mA_use);
        const float p2 = exp2f(s[n][2] - mB_use), p3 = exp2f(s[n][3] - mB_use);
        sumA += p0 + p1;
        sumB += p2 + p3;
        const int col = wtok + n * 8 + 2 * (lane & 3);
        if (warp < SW) {
          *reinterpret_cast<uint32_t*>(ps + rA * kPStride + col) = pack_bf16x2(p0, p1);
          *reinterpret_cast<uint32_t*>(ps + rB * kPStride + col) = pack_bf16x2(p2, p3);
        }
      }
      l_run[0] = l_run[0] * cA + sumA;
      l_run[1] = l_run[1] * cB + sumB;
#pragma unroll
      for (int i = 0; i < ON; ++i) { o[i][0] *= cA; o[i][1] *= cA; o[i][2] *= cB; o[i][3] *= cB; }
      math_bar();                       // the tile's probabilities are in shared memory
      if (live) {
        // O[:, (512 / MW) warp ..] += P V, V = the tile's first 512 columns
#pragma unroll
        for (int ks = 0; ks < TKM / 16; ++ks) {
          uint32_t a0, a1, a2, a3;
          ldsm4(p_addr + ks * 32, a0, a1, a2, a3);
          const int tok = ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
          for (int dn = 0; dn < ON / 2; ++dn) {
            uint32_t b0, b1, b2, b3;
            ldsm4_t(sk + lat_off(tok, warp * ON + dn * 2 + (lane >> 4)), b0, b1, b2, b3);
            mma16816(o[dn * 2], a0, a1, a2, a3, b0, b1);
            mma16816(o[dn * 2 + 1], a0, a1, a2, a3, b2, b3);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[stage]);
      }
      if (++stage == kStagesM) { stage = 0; phase ^= 1; }
    }
    // row sums: spread over the quad, and over the four warps (disjoint tokens, common maxima)
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 1);
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 2);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 1);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 2);
    if ((lane & 3) == 0) { sm_l[warp * HM + rA] = l_run[0]; sm_l[warp * HM + rB] = l_run[1]; }
    math_bar();
    float lA = 0.f, lB = 0.f;
#pragma unroll
    for (int w = 0; w < MW; ++w) { lA += sm_l[w * HM + rA]; lB += sm_l[w * HM + rB]; }
    if (split_total == 1) {
      const float iA = lA > 0.f ? 1.f / lA : 0.f, iB = lB > 0.f ? 1.f / lB : 0.f;
#pragma unroll
      for (int i = 0; i < ON; ++i) {
        const int c = warp * (DVV / MW) + i * 8 + 2 * (lane & 3);
        if (rA < valid_rows)
          *reinterpret_cast<uint32_t*>(out + (size_t)seq * out_stride + (size_t)(head0 + rA) * DVV + c) = pack_bf16x2(o[i][0] * iA, o[i][1] * iA);
        if (rB < valid_rows)
          *reinterpret_cast<uint32_t*>(out + (size_t)seq * out_stride + (size_t)(head0 + rB) * DVV + c) = pack_bf16x2(o[i][2] * iB, o[i][3] * iB);
      }
    } else {
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int r = hh ? rB : rA;
        if (r >= valid_rows) continue;
        const size_t base = ((size_t)seq * heads + head0 + r) * split_total + split_base + split;
#pragma unroll
        for (int i = 0; i < ON; ++i) {
          const int c = warp * (DVV / MW) + i * 8 + 2 * (lane & 3);
          *reinterpret_cast<float2*>(ws_o + base * DVV + c) = make_float2(o[i][2 * hh], o[i][2 * hh + 1]);
        }
        if (warp == 0 && (lane & 3) == 0) {
          ws_ml[base * 2] = m_run[hh];
          ws_ml[base * 2 + 1] = hh ? lB : lA;
        }
      }
    }
  }
  pdl_launch_dependents();
}

// ---- the steps around the attention of a latent-attention layer ----------------------------------------------------
// kern_mla_rope_append_bf16: grid = tokens, block 128. Per token: RMS-norm of the 512 compressed columns (weight w),
// rotation of the 64 positional key columns, both written as one 576-wide row of the paged latent cache at `slots[t]`;
// and the rotation, in place, of the last 64 columns of every head's 576-wide query. The rotation pairs column i with
// i + 32 (half-split), angles from the [max_pos, 32] tables.
extern "C" __global__ void __launch_bounds__(128)
    kern_mla_rope_append_bf16(const __nv_bfloat16* lat, __nv_bfloat16* q, __nv_bfloat16* cache, const long long* positions,
                              const long long* slots, const float* cos_tab, const float* sin_tab, const __nv_bfloat16* w,
                              int tokens, int heads, int lat_stride, int q_stride, float eps, long long kv_slots, int max_pos,
                              int* err) {
  __shared__ float red[4];
  pdl_wait();
  const int t = blockIdx.x;
  if (t >= tokens) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  long long pos = positions[t], slot = slots[t];
  if (pos < 0 || pos >= max_pos) { set_error(err, ERR_BOUNDS); pos = 0; }
  if (slot >= kv_slots) { set_error(err, ERR_BOUNDS); slot = -1; }
  const float* cs = cos_tab + (size_t)pos * 32;
  const float* sn = sin_tab + (size_t)pos * 32;
  const __nv_bfloat16* src = lat + (size_t)t * lat_stride;
  // the compressed part: four columns per thread
  float v[4], ss = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[j] = __bfloat162float(src[threadIdx.x * 4 + j]);
    ss += v[j] * v[j];
  }
  ss = warp_sum(ss);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  const float inv = rsqrtf((red[0] + red[1] + red[2] + red[3]) / 512.f + eps);
  if (slot >= 0) {
    __nv_bfloat16* dst = cache + (size_t)slot * DQK;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      dst[threadIdx.x * 4 + j] = __float2bfloat16(v[j] * inv * __bfloat162float(w[threadIdx.x * 4 + j]));
    if (threadIdx.x < 32) {
      const float a = __bfloat162float(src[512 + threadIdx.x]), b = __bfloat162float(src[544 + threadIdx.x]);
      dst[512 + threadIdx.x] = __float2bfloat16(a * cs[threadIdx.x] - b * sn[threadIdx.x]);
      dst[544 + threadIdx.x] = __float2bfloat16(b * cs[threadIdx.x] + a * sn[threadIdx.x]);
    }
  }
  for (int h = warp; h < heads; h += 4) {
    __nv_bfloat16* qp = q + (size_t)t * q_stride + (size_t)h * DQK + 512;
    const float a = __bfloat162float(qp[lane]), b = __bfloat162float(qp[32 + lane]);
    qp[lane] = __float2bfloat16(a * cs[lane] - b * sn[lane]);
    qp[32 + lane] = __float2bfloat16(b * cs[lane] + a * sn[lane]);
  }
}

// kern_mla_rows: grid = ceil(tokens / 128), block 128. Turns a ragged call into one attention row per token:
// row_seq[t] = the sequence of row t, row_len[t] = positions[t] + 1 (the causal reach of the row).
extern "C" __global__ void __launch_bounds__(128)
    kern_mla_rows(const long long* positions, const int* cu_q, int seqs, int tokens, int* row_seq, int* row_len) {
  pdl_wait();
  const int t = blockIdx.x * 128 + threadIdx.x;
  if (t >= tokens) return;
  int s = 0;
  while (s + 1 < seqs && t >= cu_q[s + 1]) ++s;
  row_seq[t] = s;
  row_len[t] = t < cu_q[seqs] ? (int)positions[t] + 1 : 0;
}
