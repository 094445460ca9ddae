// Paged GQA attention over the KV cache written by kern_rope_kv_append_bf16: one kernel body for
//   * decode / speculative-verify rows (few query rows per sequence; the four math warps split each
//     64-token KV tile between them, optional split-KV over grid.z with a merge kernel), and
//   * causal chunked prefill (each math warp owns 16 query rows of a 64-row block and walks the
//     KV tiles up to its causal limit; earlier chunks / a cached prefix are simply more pages).
// KV tiles are fetched by a producer warp with 2-D TMA boxes (128-byte swizzle, single-CTA destination)
// into a ring of stages guarded by bounded mbarrier waits; the math is bf16 mma.sync with f32
// online softmax. The kernel is bandwidth-bound in decode (the KV cache is read exactly once) —
// the roofline it is measured against is HBM, not the tensor cores.
// (The reference takes this kernel as a mined trtllm-gen cubin; it has no source counterpart.)
//
// Layouts: q rows live inside the fused qkv buffer (row stride q_stride elements, head h at h*D);
// out is [tokens][HQ*D]; kv pool as in attn_prep.cu; block_table [seqs][max_pages] i32;
// seq_lens [seqs] i32 = context length including this step's rows; cu_q [seqs+1] i32 row starts
// (nullptr: every sequence has rows_per_seq rows).
#include "common.cuh"

namespace kern {

constexpr int TK = 64;  // tokens per KV tile

KERN_DEVICE void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
KERN_DEVICE void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
KERN_DEVICE void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// byte offset of (token row, 16-byte chunk) inside a KV tile stored as D/64 column blocks of
// [TK rows][128 bytes] with the TMA 128-byte swizzle
KERN_DEVICE uint32_t kv_off(int tok, int chunk) {
  const int cb = chunk >> 3, c = chunk & 7;
  return (uint32_t)(cb * (TK * 128) + tok * 128 + ((c ^ (tok & 7)) << 4));
}

// Prefill with head_dim <= 128 runs a two-stage ring so that two CTAs (eight math warps) fit one SM: the row-parallel
// kernel is bound by mma.sync issue, not by the depth of its KV ring; decode keeps the deep ring (it is bandwidth-bound).
// ST > 0 fixes the depth of the ring (the ragged entry runs both kernels' CTAs side by side at two stages each).
constexpr int kAttnThreads = 160;     // the body's five warps, whatever block it runs in (a host kernel may have more and retire them)
template <int D, bool PREFILL = false, int ST = 0>
struct AttnCfg {
  static constexpr int kTileBytes = TK * D * 2;         // one of K or V
  static constexpr int kStageBytes = 2 * kTileBytes;    // K then V
  static constexpr int kStages = ST > 0 ? ST : ((PREFILL && D <= 128) ? 2 : (D >= 256 ? 3 : 4));
  static constexpr int kQStride = D + 8;                // padded bf16 row of the q tile
  static constexpr int kQBytes = 64 * kQStride * 2;
  static constexpr int kSmem = 1024 + kStages * kStageBytes + kQBytes + 256;
};

struct AttnArgs {
  const __nv_bfloat16* q;
  __nv_bfloat16* out;
  float* ws_o;       // split partials [token][hq][splits][D] (nullptr when splits == 1)
  float* ws_ml;      // [token][hq][splits][2]
  const int* block_table;
  const int* seq_lens;
  const int* cu_q;
  const int* work;        // optional work list of (sequence, query block) pairs; blockIdx.y indexes it
  const int* work_count;  // number of valid pairs
  int* err;
  int seqs, hq, hk, q_stride, out_stride, max_pages, page_size, rows_per_seq, splits, pool_pages;
  float scale_log2;
};

// PREFILL = false: decode/verify (warps split tokens); true: causal prefill (warps split rows)
// `y`: the CTA's index into the work list (or its sequence), blockIdx.y unless the caller maps it
template <int D, bool PREFILL, int ST = 0>
KERN_DEVICE void attn_body(const CUtensorMap* kv_map, const AttnArgs& a, const int y) {
  using Cfg = AttnCfg<D, PREFILL, ST>;
  constexpr int kStages = Cfg::kStages;
  constexpr int NT = PREFILL ? 8 : 2;        // 8-token n-tiles of S per warp per KV tile
  constexpr int ROWS = PREFILL ? 64 : 16;    // query rows per CTA
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* stages = smem;
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem + kStages * Cfg::kStageBytes);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * Cfg::kStageBytes + Cfg::kQBytes);
  uint64_t* empty_bar = full_bar + kStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + kStages);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = a.hq / a.hk;
  int seq = y, blk = blockIdx.x / a.hk;
  if (a.work != nullptr) {
    if (y >= *a.work_count) return;   // uniform per CTA, before any barrier
    seq = a.work[2 * y];
    blk = a.work[2 * y + 1];
  }
  const int L = a.seq_lens[seq];
  const int row0_tok = a.cu_q ? a.cu_q[seq] : seq * a.rows_per_seq;
  const int R = a.cu_q ? a.cu_q[seq + 1] - row0_tok : a.rows_per_seq;  // this step's rows
  const int toks_per_blk = PREFILL ? (64 / G) : (16 / G > 0 ? 16 / G : 1);
  const int nblk = (R + toks_per_blk - 1) / toks_per_blk;
  const int kvh = blockIdx.x % a.hk;
  const int split = blockIdx.z;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(kv_map);
  }
  __syncthreads();
  pdl_wait();
  if (blk >= nblk || L <= 0 || R <= 0) return;   // uniform per CTA

  const int tok_lo = blk * toks_per_blk;                       // first query token of this block
  const int tok_n = min(toks_per_blk, R - tok_lo);
  const int valid_rows = tok_n * G;
  // query token r (0-based among this step's R rows) sits at position L - R + r
  const int last_pos = L - R + tok_lo + tok_n - 1;
  const int ntiles_all = last_pos / TK + 1;
  // `splits` packs three numbers: bits 0-7 the KV splits of this launch, bits 8-15 the first partial slot it writes,
  // bits 16-31 the partial slots per (row, head) in the workspace (0: same as the splits). A context-parallel rank
  // writes its partials into its own run of slots of a workspace that holds every rank's; one merge covers them all.
  const int nsplit = a.splits & 0xff, split_base = (a.splits >> 8) & 0xff;
  const int split_total = (a.splits >> 16) ? (a.splits >> 16) : nsplit;
  int tile_lo = 0, tile_hi = ntiles_all;
  if (nsplit > 1) {
    const int per = (ntiles_all + nsplit - 1) / nsplit;
    tile_lo = split * per;
    tile_hi = min(ntiles_all, tile_lo + per);
    if (tile_hi < tile_lo) tile_hi = tile_lo;
  }
  const int ntiles = tile_hi - tile_lo;

  // ---- q tile -> shared (all 5 warps help) ----
  for (int i = threadIdx.x; i < ROWS * (D / 8); i += kAttnThreads) {
    const int r = i / (D / 8), c = i % (D / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < valid_rows) {
      const int tk = tok_lo + r / G, g = r % G;
      v = *reinterpret_cast<const uint4*>(a.q + (size_t)(row0_tok + tk) * a.q_stride +
                                          (size_t)(kvh * G + g) * D + c * 8);
    }
    *reinterpret_cast<uint4*>(qs + r * Cfg::kQStride + c * 8) = v;
  }
  __syncthreads();

  if (warp == 4) {
    // ---------------- producer ----------------
    if (lane == 0) {
      const int box_rows = a.page_size < TK ? a.page_size : TK;
      const int boxes = TK / box_rows;
      int stage = 0;
      uint32_t phase = 0;
      for (int t = 0; t < ntiles; ++t) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
          set_error(a.err, ERR_WAIT_EMPTY);
          *abort_flag = 1;
          break;
        }
        uint8_t* sk = stages + stage * Cfg::kStageBytes;
        uint8_t* sv = sk + Cfg::kTileBytes;
        mbar_expect_tx(&full_bar[stage], Cfg::kStageBytes);
        const int tok0 = (tile_lo + t) * TK;
        for (int b = 0; b < boxes; ++b) {
          const int tok = tok0 + b * box_rows;
          int page = 0, in_page = 0;
          const int pidx = tok / a.page_size;
          if (tok < L && pidx < a.max_pages) {
            page = a.block_table[(size_t)seq * a.max_pages + pidx];
            in_page = tok % a.page_size;
          }
          if (page < 0 || page >= a.pool_pages) {
            set_error(a.err, ERR_BOUNDS);
            page = 0;
          }
          // rows of the 2-D view: ((page*2 + kv)*HK + head)*page_size + offset
          const int krow = ((page * 2 + 0) * a.hk + kvh) * a.page_size + in_page;
          const int vrow = ((page * 2 + 1) * a.hk + kvh) * a.page_size + in_page;
#pragma unroll
          for (int cb = 0; cb < D / 64; ++cb) {
            tma_load_2d(sk + cb * (TK * 128) + b * box_rows * 128, kv_map, cb * 64, krow,
                        &full_bar[stage]);
            tma_load_2d(sv + cb * (TK * 128) + b * box_rows * 128, kv_map, cb * 64, vrow,
                        &full_bar[stage]);
          }
        }
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
    }
  }

  float o[D / 8][4];
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  if (warp < 4) {
    // ---------------- math warps ----------------
    const int qrow_base = PREFILL ? warp * 16 : 0;
    const int rA = qrow_base + (lane >> 2), rB = rA + 8;          // this thread's two rows
    const int posA = rA < valid_rows ? (L - R + tok_lo + rA / G) : -1;
    const int posB = rB < valid_rows ? (L - R + tok_lo + rB / G) : -1;
    const uint32_t q_addr = smem_u32(qs) + ((qrow_base + (lane & 7) + ((lane >> 3) & 1) * 8) *
                                            Cfg::kQStride + (lane >> 4) * 8) * 2;
    int stage = 0;
    uint32_t phase = 0;
    for (int t = 0; t < ntiles; ++t) {
      if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
        set_error(a.err, ERR_WAIT_FULL);
        *abort_flag = 1;
        break;
      }
      const uint32_t sk = smem_u32(stages + stage * Cfg::kStageBytes);
      const uint32_t sv = sk + Cfg::kTileBytes;
      const int tok0 = (tile_lo + t) * TK;
      const int wtok = PREFILL ? 0 : warp * 16;   // this warp's token offset inside the tile
      // a whole tile above the causal limit of this warp's rows contributes nothing
      const int warp_max_pos = L - R + tok_lo + min(valid_rows - 1, qrow_base + 15) / G;
      const bool skip = PREFILL && (tok0 > warp_max_pos || qrow_base >= valid_rows);
      if (!skip) {
        // ---- S = Q K^T ----
        float s[NT][4];
#pragma unroll
        for (int n = 0; n < NT; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < D / 16; kk += 2) {
          uint32_t qa[2][4];
          ldsm_x4(q_addr + kk * 32, qa[0][0], qa[0][1], qa[0][2], qa[0][3]);
          ldsm_x4(q_addr + kk * 32 + 32, qa[1][0], qa[1][1], qa[1][2], qa[1][3]);
#pragma unroll
          for (int n = 0; n < NT; ++n) {
            // four 8x8 matrices: tokens n*8.., d chunks 2kk .. 2kk+3
            const int tok = wtok + n * 8 + (lane & 7);
            uint32_t b0, b1, b2, b3;
            ldsm_x4(sk + kv_off(tok, kk * 2 + (lane >> 3)), b0, b1, b2, b3);
            mma_bf16_16816(s[n], qa[0][0], qa[0][1], qa[0][2], qa[0][3], b0, b1);
            mma_bf16_16816(s[n], qa[1][0], qa[1][1], qa[1][2], qa[1][3], b2, b3);
          }
        }
        // ---- mask + online softmax (base-2) ----
        float mxA = -INFINITY, mxB = -INFINITY;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          const int j = tok0 + wtok + n * 8 + 2 * (lane & 3);
          s[n][0] = (j <= posA) ? s[n][0] * a.scale_log2 : -INFINITY;
          s[n][1] = (j + 1 <= posA) ? s[n][1] * a.scale_log2 : -INFINITY;
          s[n][2] = (j <= posB) ? s[n][2] * a.scale_log2 : -INFINITY;
          s[n][3] = (j + 1 <= posB) ? s[n][3] * a.scale_log2 : -INFINITY;
          mxA = fmaxf(mxA, fmaxf(s[n][0], s[n][1]));
          mxB = fmaxf(mxB, fmaxf(s[n][2], s[n][3]));
        }
        mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1));
        mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
        mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1));
        mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
        const float mA = fmaxf(m_run[0], mxA), mB = fmaxf(m_run[1], mxB);
        const float mA_use = mA == -INFINITY ? 0.f : mA, mB_use = mB == -INFINITY ? 0.f : mB;
        const float cA = exp2f(m_run[0] - mA_use), cB = exp2f(m_run[1] - mB_use);
        m_run[0] = mA;
        m_run[1] = mB;
        float sumA = 0.f, sumB = 0.f;
        uint32_t pa[NT][2];
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          const float p0 = exp2f(s[n][0] - mA_use), p1 = exp2f(s[n][1] - mA_use);
          const float p2 = exp2f(s[n][2] - mB_use), p3 = exp2f(s[n][3] - mB_use);
          sumA += p0 + p1;
          sumB += p2 + p3;
          pa[n][0] = pack_bf16x2(p0, p1);
          pa[n][1] = pack_bf16x2(p2, p3);
        }
        l_run[0] = l_run[0] * cA + sumA;
        l_run[1] = l_run[1] * cB + sumB;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
          o[i][0] *= cA; o[i][1] *= cA; o[i][2] *= cB; o[i][3] *= cB;
        }
        // ---- O += P V ----
#pragma unroll
        for (int ks = 0; ks < NT / 2; ++ks) {   // 16 tokens per k-step
          const int tok = wtok + ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
          for (int dn = 0; dn < D / 16; ++dn) {  // two 8-wide d tiles per ldmatrix.x4.trans
            uint32_t b0, b1, b2, b3;
            ldsm_x4_t(sv + kv_off(tok, dn * 2 + (lane >> 4)), b0, b1, b2, b3);
            mma_bf16_16816(o[dn * 2], pa[2 * ks][0], pa[2 * ks][1], pa[2 * ks + 1][0],
                           pa[2 * ks + 1][1], b0, b1);
            mma_bf16_16816(o[dn * 2 + 1], pa[2 * ks][0], pa[2 * ks][1], pa[2 * ks + 1][0],
                           pa[2 * ks + 1][1], b2, b3);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[stage]);
      if (++stage == kStages) { stage = 0; phase ^= 1; }
    }
    // row sums live spread over the quad
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 1);
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 2);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 1);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 2);
  }

  // ---------------- combine + write ----------------
  if (!PREFILL) {
    // the four warps hold partial (m, l, O) of the same 16 rows over disjoint tokens: merge in smem
    __syncthreads();  // every stage has been consumed: reuse the stage memory
    float* mo = reinterpret_cast<float*>(stages);            // [4][16][D]
    float* mm = mo + 4 * 16 * D;                             // [4][16]
    float* ml = mm + 64;                                     // [4][16]
    if (warp < 4) {
      const int rA = lane >> 2, rB = rA + 8;
      if ((lane & 3) == 0) {
        mm[warp * 16 + rA] = m_run[0]; mm[warp * 16 + rB] = m_run[1];
        ml[warp * 16 + rA] = l_run[0]; ml[warp * 16 + rB] = l_run[1];
      }
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        const int c = i * 8 + 2 * (lane & 3);
        *reinterpret_cast<float2*>(mo + (warp * 16 + rA) * D + c) = make_float2(o[i][0], o[i][1]);
        *reinterpret_cast<float2*>(mo + (warp * 16 + rB) * D + c) = make_float2(o[i][2], o[i][3]);
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 16 * D; i += kAttnThreads) {
      const int r = i / D, c = i % D;
      if (r >= valid_rows) continue;
      float m = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) m = fmaxf(m, mm[w * 16 + r]);
      const float m_use = m == -INFINITY ? 0.f : m;
      float l = 0.f, acc = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float f = exp2f(mm[w * 16 + r] - m_use);
        l += ml[w * 16 + r] * f;
        acc += mo[(w * 16 + r) * D + c] * f;
      }
      const int tk = row0_tok + tok_lo + r / G, head = kvh * G + r % G;
      if (split_total == 1) {
        a.out[(size_t)tk * a.out_stride + (size_t)head * D + c] =
            __float2bfloat16(l > 0.f ? acc / l : 0.f);
      } else {
        const size_t base = ((size_t)tk * a.hq + head) * split_total + split_base + split;
        a.ws_o[base * D + c] = acc;
        if (c == 0) {
          a.ws_ml[base * 2] = m;
          a.ws_ml[base * 2 + 1] = l;
        }
      }
    }
  } else if (warp < 4) {
    const int rA = warp * 16 + (lane >> 2), rB = rA + 8;
    const float iA = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f, iB = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      const int c = i * 8 + 2 * (lane & 3);
      if (rA < valid_rows) {
        const int tk = row0_tok + tok_lo + rA / G, head = kvh * G + rA % G;
        *reinterpret_cast<uint32_t*>(a.out + (size_t)tk * a.out_stride + (size_t)head * D + c) =
            pack_bf16x2(o[i][0] * iA, o[i][1] * iA);
      }
      if (rB < valid_rows) {
        const int tk = row0_tok + tok_lo + rB / G, head = kvh * G + rB % G;
        *reinterpret_cast<uint32_t*>(a.out + (size_t)tk * a.out_stride + (size_t)head * D + c) =
            pack_bf16x2(o[i][2] * iB, o[i][3] * iB);
      }
    }
  }
  pdl_launch_dependents();
}

}  // namespace kern

#ifndef KERN_ATTN_NO_ENTRIES      // a file that includes this one for attn_body alone defines it
using namespace kern;

#define KERN_ATTN_ENTRY(name, D, PREFILL)                                                        \
  extern "C" __global__ void __launch_bounds__(160, (PREFILL && D <= 128) ? 2 : 1)               \
      name(const __grid_constant__ CUtensorMap kv_map, const __nv_bfloat16* q,                   \
           __nv_bfloat16* out, float* ws_o, float* ws_ml, const int* block_table,                \
           const int* seq_lens, const int* cu_q, const int* work, const int* work_count,         \
           int seqs, int hq, int hk, int q_stride,                                               \
           int out_stride, int max_pages, int page_size, int rows_per_seq, int splits,           \
           int pool_pages, float scale_log2, int* err) {                                         \
    AttnArgs a{q, out, ws_o, ws_ml, block_table, seq_lens, cu_q, work, work_count, err, seqs, hq, \
               hk, q_stride,                                                                     \
               out_stride, max_pages, page_size, rows_per_seq, splits, pool_pages, scale_log2};  \
    attn_body<D, PREFILL>(&kv_map, a, (int)blockIdx.y);                                          \
  }

KERN_ATTN_ENTRY(kern_attn_decode_paged_d64, 64, false)
KERN_ATTN_ENTRY(kern_attn_decode_paged_d128, 128, false)
KERN_ATTN_ENTRY(kern_attn_decode_paged_d256, 256, false)
KERN_ATTN_ENTRY(kern_attn_prefill_paged_d64, 64, true)
KERN_ATTN_ENTRY(kern_attn_prefill_paged_d128, 128, true)
KERN_ATTN_ENTRY(kern_attn_prefill_paged_d256, 256, true)

// Both lists of a ragged call in one launch (head_dim <= 128): CTAs of the row-parallel causal kernel (list p, bound by
// tensor-core issue) and of the token-parallel kernel (list d, bound by the KV stream) alternate in launch order while
// both lists last, two CTAs per SM with a two-stage ring each, so the decode rows' KV streams while the prompt rows'
// tiles compute. grid = (hk, at least count_p + count_d).
#define KERN_ATTN_RAGGED_ENTRY(name, D)                                                          \
  extern "C" __global__ void __launch_bounds__(160, 2)                                           \
      name(const __grid_constant__ CUtensorMap kv_map, const __nv_bfloat16* q,                   \
           __nv_bfloat16* out, const int* block_table, const int* seq_lens, const int* cu_q,     \
           const int* work_p, const int* count_p, const int* work_d, const int* count_d,         \
           int hq, int hk, int q_stride, int out_stride, int max_pages, int page_size,           \
           int pool_pages, float scale_log2, int* err) {                                         \
    const int np = *count_p, nd = *count_d, m = np < nd ? np : nd;                               \
    const int y = blockIdx.y;                                                                    \
    if (y >= np + nd) return;                                                                    \
    const bool is_p = y < 2 * m ? !(y & 1) : np > nd;                                            \
    const int idx = y < 2 * m ? (y >> 1) : y - m;                                                \
    AttnArgs a{q, out, nullptr, nullptr, block_table, seq_lens, cu_q, is_p ? work_p : work_d,    \
               is_p ? count_p : count_d, err, 0x7fffffff, hq, hk, q_stride, out_stride,          \
               max_pages, page_size, 1, 1, pool_pages, scale_log2};                              \
    if (is_p) attn_body<D, true, 2>(&kv_map, a, idx);                                            \
    else attn_body<D, false, 2>(&kv_map, a, idx);                                                \
  }

KERN_ATTN_RAGGED_ENTRY(kern_attn_ragged_paged_d64, 64)
KERN_ATTN_RAGGED_ENTRY(kern_attn_ragged_paged_d128, 128)

// Work lists for a ragged call: one (sequence, query block) pair per block of new rows, so the
// attention grids are sized by the rows of the call and not by sequences x the longest one.
// Sequences with at most `small_rows` new rows (decode rows and speculative rounds riding in a ragged
// batch) go to list d in blocks of `tpb_d` tokens for the token-parallel kernel, where four warps share
// each KV tile; the rest go to list p in blocks of `tpb_p` tokens for the row-parallel causal kernel.
// One CTA; the plan is the same for every layer of a step.
extern "C" __global__ void kern_attn_plan(const int* cu_q, int seqs, int tpb_p, int tpb_d, int small_rows,
                                          int* work_p, int* count_p, int max_p, int* work_d,
                                          int* count_d, int max_d) {
  pdl_wait();
  __shared__ int base_p[1025], base_d[1025];
  if (threadIdx.x == 0) {
    int np = 0, nd = 0;
    for (int s = 0; s < seqs && s < 1024; ++s) {
      base_p[s] = np;
      base_d[s] = nd;
      const int r = cu_q[s + 1] - cu_q[s];
      if (r <= 0) continue;
      if (r <= small_rows) nd += (r + tpb_d - 1) / tpb_d;
      else np += (r + tpb_p - 1) / tpb_p;
    }
    const int e = seqs < 1024 ? seqs : 1024;
    base_p[e] = np;
    base_d[e] = nd;
    *count_p = np < max_p ? np : max_p;
    *count_d = nd < max_d ? nd : max_d;
  }
  __syncthreads();
  for (int s = threadIdx.x; s < seqs && s < 1024; s += blockDim.x) {
    for (int i = base_p[s]; i < base_p[s + 1] && i < max_p; ++i) {
      work_p[2 * i] = s;
      work_p[2 * i + 1] = i - base_p[s];
    }
    for (int i = base_d[s]; i < base_d[s + 1] && i < max_d; ++i) {
      work_d[2 * i] = s;
      work_d[2 * i + 1] = i - base_d[s];
    }
  }
}

// Merge split-KV partials: out[token][head][:] = sum_s O_s * 2^(m_s - m) / sum_s l_s * 2^(m_s - m)
// grid = tokens * hq, block = D threads (<= 256)
extern "C" __global__ void kern_attn_merge_splits(const float* ws_o, const float* ws_ml,
                                                  __nv_bfloat16* out, int rows, int hq, int d,
                                                  int splits, int out_stride) {
  pdl_wait();
  const int row = blockIdx.x;  // token * hq + head
  if (row >= rows) return;
  const int tk = row / hq, head = row % hq;
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, ws_ml[((size_t)row * splits + s) * 2]);
  const float m_use = m == -INFINITY ? 0.f : m;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float l = 0.f, acc = 0.f;
    for (int s = 0; s < splits; ++s) {
      const size_t b = (size_t)row * splits + s;
      const float f = exp2f(ws_ml[b * 2] - m_use);
      l += ws_ml[b * 2 + 1] * f;
      acc += ws_o[b * d + c] * f;
    }
    out[(size_t)tk * out_stride + (size_t)head * d + c] = __float2bfloat16(l > 0.f ? acc / l : 0.f);
  }
}

// Merge the partials of a context-parallel group after an all-gather: rank r's compact workspace ([rows * hq][splits]
// slots, as a launch with `partial = (0, splits)` writes it) sits at ws + r * rows * splits slots. Same arithmetic as
// above over ranks * splits slots. grid = tokens * hq, block = D threads (<= 256).
extern "C" __global__ void kern_attn_merge_ranks(const float* ws_o, const float* ws_ml, __nv_bfloat16* out, int rows, int hq,
                                                 int d, int splits, int ranks, int out_stride) {
  pdl_wait();
  const int row = blockIdx.x;  // token * hq + head
  if (row >= rows) return;
  const int tk = row / hq, head = row % hq;
  float m = -INFINITY;
  for (int r = 0; r < ranks; ++r)
    for (int s = 0; s < splits; ++s) m = fmaxf(m, ws_ml[(((size_t)r * rows + row) * splits + s) * 2]);
  const float m_use = m == -INFINITY ? 0.f : m;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float l = 0.f, acc = 0.f;
    for (int r = 0; r < ranks; ++r)
      for (int s = 0; s < splits; ++s) {
        const size_t b = ((size_t)r * rows + row) * splits + s;
        const float f = exp2f(ws_ml[b * 2] - m_use);
        l += ws_ml[b * 2 + 1] * f;
        acc += ws_o[b * d + c] * f;
      }
    out[(size_t)tk * out_stride + (size_t)head * d + c] = __float2bfloat16(l > 0.f ? acc / l : 0.f);
  }
}

// Context parallel by position: position p of a sequence lives on member p % world at local index p / world, so a
// sequence of L positions has ceil((L - rank) / world) of them here. grid = ceil(seqs / 256), block 256.
extern "C" __global__ void kern_dcp_local_lens(const int* seq_lens, int* local_lens, int seqs, int rank, int world) {
  pdl_wait();
  const int s = blockIdx.x * 256 + threadIdx.x;
  if (s >= seqs) return;
  const int L = seq_lens[s];
  local_lens[s] = L > rank ? (L - rank + world - 1) / world : 0;
}


// Start of a context-parallel decode attention: the local length of every sequence, and every partial slot of the
// call set neutral (m = -inf, l = 0) so that a member whose share of a sequence is empty contributes nothing.
// grid = seqs, block 128; slots = heads * splits partial slots per sequence row.
extern "C" __global__ void __launch_bounds__(128)
    kern_dcp_prepare(const int* seq_lens, int* local_lens, float* ws_ml, int seqs, int rank, int world, int slots) {
  pdl_wait();
  const int s = blockIdx.x;
  if (s >= seqs) return;
  if (threadIdx.x == 0) {
    const int L = seq_lens[s];
    local_lens[s] = L > rank ? (L - rank + world - 1) / world : 0;
  }
  for (int i = threadIdx.x; i < slots; i += 128)
    *reinterpret_cast<float2*>(ws_ml + ((size_t)s * slots + i) * 2) = make_float2(-INFINITY, 0.f);
}

// Deal the rows of a paged KV pool to a member of a by-position group: local index li of sequence s on member `rank`
// is position li * world + rank. Copies K and V rows (all kv heads) from the source pool (the whole context, this
// GPU's) into the destination pool (the member's, possibly another GPU's memory mapped here: plain 16-byte stores).
// KV layout of both: [page][k|v][kv_head][page_size][head_dim] bf16. grid [ceil(max local rows / 4), seqs], block 128:
// a warp per row. Tables: [seqs][width] page ids; src_lens = whole lengths.
// Reference counterpart: crates/kern-runtime/src/push.rs:398-434 (push_rows), :494 (the gather kernel).
extern "C" __global__ void __launch_bounds__(128)
    kern_deal_rows_bf16(const __nv_bfloat16* src, __nv_bfloat16* dst, const int* src_table, const int* dst_table,
                        const int* src_lens, int seqs, int src_width, int dst_width, int hk, int d, int page_size, int rank,
                        int world, int first_pos, int* err) {
  pdl_wait();
  const int s = blockIdx.y;
  if (s >= seqs) return;
  const int li = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  const int L = src_lens[s];
  const long long pos = (long long)li * world + rank;
  if (pos >= L || pos < first_pos) return;      // first_pos: rows below it were dealt by an earlier call
  const int sp = (int)(pos / page_size), so = (int)(pos % page_size), dp = li / page_size, dof = li % page_size;
  if (sp >= src_width || dp >= dst_width) {
    if (lane == 0) set_error(err, ERR_BOUNDS);
    return;
  }
  const size_t page_elems = (size_t)2 * hk * page_size * d;
  const __nv_bfloat16* sb = src + (size_t)src_table[(size_t)s * src_width + sp] * page_elems + (size_t)so * d;
  __nv_bfloat16* db = dst + (size_t)dst_table[(size_t)s * dst_width + dp] * page_elems + (size_t)dof * d;
  const int vecs = d / 8;
  for (int i = lane; i < 2 * hk * vecs; i += 32) {
    const int blk = i / vecs, v = i % vecs;      // blk = (k|v) * hk + head
    reinterpret_cast<uint4*>(db + (size_t)blk * page_size * d)[v] =
        reinterpret_cast<const uint4*>(sb + (size_t)blk * page_size * d)[v];
  }
}
#endif  // KERN_ATTN_NO_ENTRIES
