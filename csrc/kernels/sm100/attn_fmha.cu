// Causal prefill attention over the paged KV cache on the 5th-generation tensor cores (head_dim 128).
//
// One CTA = one (sequence, block of query rows, KV head): 128 query rows (128 / G tokens x the G query heads that
// share the KV head), walked over KV tiles of 128 tokens up to the block's causal limit:
//
//   warp 0      TMA producer: K and V tiles of the paged cache (2-D boxes per page, 128-byte swizzle) into a ring
//   warp 1      issues the MMAs from one thread:  S = Q K^T   (128 x 128 x D, accumulator in TMEM, two S buffers)
//                                                 O += P V    (128 x D x 128, accumulator in TMEM)
//   warps 2..5  softmax, one thread per query row: read its row of S out of TMEM (tcgen05.ld), running maximum,
//               exponentials, row sum, and P as bf16 into shared memory (the A operand of the second MMA);
//               at the end read O, divide by the row sum and store
//
// S(j + 1) = Q K^T is issued before P(j) V, so the tensor cores work on the next tile's scores while the softmax
// warps are busy with this tile's. O is rescaled lazily: a row's reference maximum moves only when the running
// maximum has grown by more than 8 (a factor 256, harmless in f32), so most tiles need no pass over O at all.
// V is consumed straight from its [token][d] tile as an MN-major B operand: no transpose anywhere.
// Every mbarrier wait is bounded by wall-clock time (2 s); a wait that runs out sets *err with the code of the wait
// that gave up, the CTA drains and frees its TMEM.
//
// Layouts as in attn_paged.cu (q rows inside the fused qkv buffer; kv pool [pages][2][hk][page][d] behind one 2-D
// tensor map with 64-column boxes; block_table, seq_lens, cu_q, the planner's work list).
// The reference takes prefill attention as a prebuilt trtllm-gen FMHA blob (kernel_index/trtllm_fmha_*.toml); it has no
// source counterpart.
#define KERN_ATTN_NO_ENTRIES
#include "attn_paged.cu"      // attn_body: the token-parallel kernel that shares an SM with this one in the ragged entry

namespace kern {

constexpr int FM = 128;   // query rows per CTA
// FN, the tokens per KV tile, is a template parameter: 128 (one CTA per SM: all 512 TMEM columns, 193 KB of shared
// memory) or 64 (S buffers of 64 columns: 256 TMEM columns and 113 KB, so two CTAs share an SM and one's MMAs run under
// the other's softmax, which is the critical path of this kernel).

// Shared-memory descriptor of an MN-major operand tile written by TMA with the 128-byte swizzle: rows are K (tokens),
// each 128 bytes = 64 MN elements; 8 rows form a 1024-byte swizzle atom; the next 64 MN elements are `mn_block_bytes`
// further on.
KERN_DEVICE uint64_t umma_desc_sw128_mn(uint32_t smem_addr, uint32_t mn_block_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((mn_block_bytes >> 4) & 0x3FFF) << 16;   // leading byte offset: next block of 64 along MN
  d |= (uint64_t)(1024 >> 4) << 32;                        // stride byte offset: next 8 rows along K
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;                                  // SWIZZLE_128B
  return d;
}

KERN_DEVICE void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
KERN_DEVICE void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

template <int D, int FN>
struct FmhaCfg {
  static constexpr int kQBytes = FM * D * 2;              // D / 64 column blocks of [128 rows][128 bytes]
  static constexpr int kPBytes = FM * FN * 2;             // FN / 64 blocks of 64 tokens
  static constexpr int kTileBytes = FN * D * 2;           // K or V
  static constexpr int kStages = 2;
  // room to bring the tiles to a 1024-byte boundary: the two-per-SM form has 768 bytes to spare under the SM's 228 KB
  // and checks that its (1024-aligned in practice) base needs no more
  static constexpr int kSlack = FN == 64 ? 768 : 1024;
  static constexpr int kSmem = kSlack + kQBytes + kPBytes + kStages * 2 * kTileBytes + 256;
  static constexpr int kTmemCols = 2 * FN + D <= 256 ? 256 : 512;   // S0 | S1 | O
};

struct FmhaArgs {
  const __nv_bfloat16* q;
  __nv_bfloat16* out;
  const int* block_table;
  const int* seq_lens;
  const int* cu_q;
  const int* work;
  const int* work_count;
  int* err;
  int hq, hk, q_stride, out_stride, max_pages, page_size, pool_pages;
  float scale_log2;
};

// `y`: the CTA's index into the work list (blockIdx.y unless the caller maps it)
template <int D, int FN>
KERN_DEVICE void fmha_body(const CUtensorMap* kv_map, const FmhaArgs& a, const int y) {
  using Cfg = FmhaCfg<D, FN>;
  constexpr int kStages = Cfg::kStages;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  if ((int)(smem - smem_raw) > Cfg::kSlack) {             // uniform per CTA, before any barrier or allocation
    if (threadIdx.x == 0) set_error(a.err, ERR_BOUNDS);
    return;
  }
  uint8_t* q_s = smem;
  uint8_t* p_s = q_s + Cfg::kQBytes;
  uint8_t* kv_s = p_s + Cfg::kPBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(kv_s + kStages * 2 * Cfg::kTileBytes);
  // K and V of a stage have barriers of their own: a stage's K half is free as soon as Q K^T has read it — a whole tile
  // period before P V lets go of the V half — so the load of the K tile after next starts that much earlier and Q K^T
  // never waits for a load that was only just issued.
  uint64_t* k_full = bars;                   // [stages]  TMA -> MMA (K half)
  uint64_t* v_full = k_full + kStages;       // [stages]  TMA -> MMA (V half)
  uint64_t* k_empty = v_full + kStages;      // [stages]  Q K^T done with the K half
  uint64_t* v_empty = k_empty + kStages;     // [stages]  P V done with the V half
  uint64_t* s_full = v_empty + kStages;      // [2]       S buffer written
  uint64_t* s_empty = s_full + 2;            // [2]       softmax has read the S buffer (128 arrivals)
  uint64_t* p_full = s_empty + 2;            // [1]       P in shared memory (128 arrivals)
  uint64_t* p_empty = p_full + 1;            // [1]       P V has consumed P (and O is quiet)
  uint64_t* o_full = p_empty + 1;            // [1]       last P V done
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = a.hq / a.hk;
  if (y >= *a.work_count) return;          // uniform per CTA, before any barrier or allocation
  if (*reinterpret_cast<volatile int*>(a.err) != 0) return;   // an earlier CTA (or kernel) gave up: the call is lost, do not wait again
  const int seq = a.work[2 * y], blk = a.work[2 * y + 1];
  const int kvh = blockIdx.x;
  const int L = a.seq_lens[seq];
  const int row0_tok = a.cu_q[seq];
  const int R = a.cu_q[seq + 1] - row0_tok;
  const int toks_per_blk = FM / G;
  const int tok_lo = blk * toks_per_blk;
  if (tok_lo >= R || L <= 0) return;
  const int tok_n = min(toks_per_blk, R - tok_lo);
  const int valid_rows = tok_n * G;
  const int last_pos = L - R + tok_lo + tok_n - 1;
  const int ntiles = last_pos / FN + 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&v_full[s], 1);
      mbar_init(&k_empty[s], 1); mbar_init(&v_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) { mbar_init(&s_full[b], 1); mbar_init(&s_empty[b], 128); }
    mbar_init(p_full, 128);
    mbar_init(p_empty, 1);
    mbar_init(o_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(kv_map);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();

  // ---- Q tile -> shared memory in the K-major 128-byte-swizzled layout the MMA reads (all warps) ----
  for (int i = threadIdx.x; i < FM * (D / 8); i += blockDim.x) {
    const int r = i / (D / 8), c = i % (D / 8);            // row, 16-byte chunk
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < valid_rows) {
      const int tk = tok_lo + r / G, g = r % G;
      v = *reinterpret_cast<const uint4*>(a.q + (size_t)(row0_tok + tk) * a.q_stride + (size_t)(kvh * G + g) * D + c * 8);
    }
    const int cb = c >> 3, cc = c & 7;
    *reinterpret_cast<uint4*>(q_s + cb * (FM * 128) + r * 128 + ((cc ^ (r & 7)) << 4)) = v;
  }
  fence_proxy_async();        // generic-proxy stores above are read by the tensor core's async proxy
  __syncthreads();

  if (warp == 0) {
    // ---------------- producer ----------------
    if (lane == 0) {
      const int box_rows = a.page_size < 64 ? a.page_size : 64;
      const int boxes = FN / box_rows;
      // one half (K: which = 0, V: which = 1) of tile t into its stage, behind the half's own empty barrier
      auto load_half = [&](int t, int which) -> bool {
        const int stage = t % kStages;
        const uint32_t parity = ((t / kStages) & 1) ^ 1;
        uint64_t* empty = which ? &v_empty[stage] : &k_empty[stage];
        uint64_t* full = which ? &v_full[stage] : &k_full[stage];
        if (!mbar_wait_ns(empty, parity, abort_flag)) {
          set_error(a.err, ERR_WAIT_EMPTY);
          *abort_flag = 1;
          return false;
        }
        uint8_t* dst = kv_s + stage * 2 * Cfg::kTileBytes + which * Cfg::kTileBytes;
        mbar_expect_tx(full, Cfg::kTileBytes);
        for (int b = 0; b < boxes; ++b) {
          const int tok = t * FN + b * box_rows;
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
          const int row = ((page * 2 + which) * a.hk + kvh) * a.page_size + in_page;
#pragma unroll
          for (int cb = 0; cb < D / 64; ++cb)
            tma_load_2d(dst + cb * (FN * 128) + b * box_rows * 128, kv_map, cb * 64, row, full);
        }
        return true;
      };
      // issue order K(0), then for every tile K(t + 1) before V(t): the waits then come in the order the MMAs complete
      // (Q K^T of tile t - 1 is issued before P V of tile t - 2)
      bool ok = load_half(0, 0);
      for (int t = 0; t < ntiles && ok; ++t) {
        if (t + 1 < ntiles) ok = load_half(t + 1, 0);
        if (ok) ok = load_half(t, 1);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(FM, FN);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(FM, D) | (1u << 16);      // B (= V) is MN-major
      const uint32_t o_tmem = tmem_base + 2 * FN;
      bool ok = true;
      auto issue_qk = [&](int j) {
        const int stage = j % kStages;
        if (!mbar_wait_ns(&k_full[stage], (j / kStages) & 1, abort_flag)) { set_error(a.err, ERR_WAIT_FULL); return false; }
        if (!mbar_wait_ns(&s_empty[j & 1], ((j >> 1) & 1) ^ 1, abort_flag)) { set_error(a.err, ERR_WAIT_TMEM_EMPTY); return false; }
        tc_fence_after();
        const uint32_t sq = smem_u32(q_s), sk = smem_u32(kv_s + stage * 2 * Cfg::kTileBytes);
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          umma_bf16(tmem_base + (j & 1) * FN, umma_desc_sw128(sq + (k >> 2) * (FM * 128) + (k & 3) * 32),
                    umma_desc_sw128(sk + (k >> 2) * (FN * 128) + (k & 3) * 32), idesc_qk, k != 0);
        tc_commit(&s_full[j & 1]);
        tc_commit(&k_empty[stage]);         // the K half is free once these MMAs have read it
        return true;
      };
      auto issue_pv = [&](int j) {
        const int stage = j % kStages;
        if (!mbar_wait_ns(&v_full[stage], (j / kStages) & 1, abort_flag)) { set_error(a.err, ERR_WAIT_FULL); return false; }
        if (!mbar_wait_ns(p_full, j & 1, abort_flag)) { set_error(a.err, ERR_WAIT_FULL); return false; }
        tc_fence_after();
        const uint32_t sp = smem_u32(p_s), sv = smem_u32(kv_s + stage * 2 * Cfg::kTileBytes + Cfg::kTileBytes);
#pragma unroll
        for (int k = 0; k < FN / 16; ++k)
          umma_bf16(o_tmem, umma_desc_sw128(sp + (k >> 2) * (FM * 128) + (k & 3) * 32),
                    umma_desc_sw128_mn(sv + k * 16 * 128, FN * 128), idesc_pv, (j | k) != 0);
        tc_commit(&v_empty[stage]);         // the V half of the stage is free
        tc_commit(p_empty);                 // P is consumed and O is quiet until the next P V
        if (j == ntiles - 1) tc_commit(o_full);
        return true;
      };
      ok = issue_qk(0);
      for (int j = 0; j < ntiles && ok; ++j) {
        if (j + 1 < ntiles) ok = issue_qk(j + 1);     // next tile's scores first: they overlap this tile's softmax
        if (ok) ok = issue_pv(j);
      }
      if (!ok) *abort_flag = 1;
    }
    __syncwarp();
  } else {
    // ---------------- softmax warps 2..5: one thread per query row ----------------
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;                           // row of the tile = TMEM lane
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const int pos = row < valid_rows ? (L - R + tok_lo + row / G) : -1;       // last token this row may attend to
    float m_ref = -INFINITY, l_run = 0.f;                          // reference maximum (lazy) and row sum
    bool ok = true;
    for (int j = 0; j < ntiles && ok; ++j) {
      if (!mbar_wait_ns(&s_full[j & 1], (j >> 1) & 1, abort_flag)) { set_error(a.err, ERR_WAIT_TMEM_FULL); *abort_flag = 1; ok = false; break; }
      tc_fence_after();
      const uint32_t s_tmem = tmem_base + lane_addr + (j & 1) * FN;
      const int tok0 = j * FN;
      const bool diag = tok0 + FN - 1 > pos;                        // some column of the tile is above this row's limit
      // pass 1: the row maximum of the tile. With 64-token tiles the row's 64 scores stay in registers for pass 2 (one
      // read of S instead of two), and the S buffer is handed back to the MMA warp at once.
      constexpr bool kKeep = FN <= 64;
      uint32_t keep[kKeep ? FN : 1];
      float mx = -INFINITY;
      if constexpr (kKeep) {
#pragma unroll
        for (int c = 0; c < FN / 32; ++c) tmem_ld_32x32(s_tmem + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&keep[c * 32]));
        tmem_ld_wait();
        if (diag) {       // the causal limit, once, on the scores themselves (a per-row branch: no warp-wide instruction inside)
#pragma unroll
          for (int i = 0; i < FN; ++i)
            if (tok0 + i > pos) keep[i] = 0xff800000u;      // -inf
        }
        {
          float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};      // four chains: a single one is 64 dependent steps
#pragma unroll
          for (int i = 0; i < FN; ++i) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(keep[i]));
          mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
        }
        tc_fence_before();
        mbar_arrive(&s_empty[j & 1]);
      } else {
#pragma unroll 1
        for (int c = 0; c < FN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(s_tmem + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (!diag || tok0 + c * 32 + i <= pos) mx = fmaxf(mx, __uint_as_float(r[i]));
        }
      }
      mx *= a.scale_log2;
      // lazy reference maximum: move it (and rescale O and l) only when the running maximum outgrew it by 2^8
      float alpha = 1.f;
      bool moved = false;
      if (mx > m_ref + 8.f) {
        alpha = m_ref == -INFINITY ? 0.f : exp2f(m_ref - mx);
        m_ref = mx;
        moved = true;
      }
      // P and O may be touched once P(j-1) V is done
      if (j > 0 && !mbar_wait_ns(p_empty, (j - 1) & 1, abort_flag)) { set_error(a.err, ERR_WAIT_EMPTY); *abort_flag = 1; ok = false; break; }
      tc_fence_after();
      // tcgen05.ld / st are warp-wide (.sync.aligned): the pass over O runs for the whole warp when any of its rows
      // moved (alpha is 1 for the rows that did not), never under a per-lane branch
      if (__any_sync(0xffffffffu, moved && j > 0)) {
        const uint32_t o_tmem = tmem_base + lane_addr + 2 * FN;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(o_tmem + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st_32x32(o_tmem + c * 32, r);
        }
        tmem_st_wait();
      }
      l_run *= alpha;
      // pass 2: exponentials -> P (bf16, K-major swizzled, the A operand of P V), row sum
      const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
      float sum = 0.f, sum_b = 0.f;
#pragma unroll
      for (int c = 0; c < FN / 32; ++c) {
        uint32_t r[32];
        if constexpr (kKeep) {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = keep[c * 32 + i];
        } else {
          tmem_ld_32x32(s_tmem + c * 32, r);
          tmem_ld_wait();
        }
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int t = tok0 + c * 32 + 2 * i;
          // (kept scores carry the causal limit already: a masked one is -inf and its exponential 0)
          const float p0 = (kKeep || !diag || t <= pos) ? exp2f(__uint_as_float(r[2 * i]) * a.scale_log2 - m_use) : 0.f;
          const float p1 = (kKeep || !diag || t + 1 <= pos) ? exp2f(__uint_as_float(r[2 * i + 1]) * a.scale_log2 - m_use) : 0.f;
          if (i & 1) sum_b += p0 + p1; else sum += p0 + p1;
          pk[i] = pack_bf16x2(p0, p1);
        }
        // 32 tokens = four 16-byte chunks of this row: chunks 4c .. 4c+3 of 16, block (4c) >> 3
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int chunk = c * 4 + q, cb = chunk >> 3, cc = chunk & 7;
          *reinterpret_cast<uint4*>(p_s + cb * (FM * 128) + row * 128 + ((cc ^ (row & 7)) << 4)) =
              make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
        }
      }
      l_run += sum + sum_b;
      tc_fence_before();
      fence_proxy_async();
      if constexpr (!kKeep) mbar_arrive(&s_empty[j & 1]);
      mbar_arrive(p_full);
    }
    // ---- epilogue: O / l -> out ----
    if (ok && !mbar_wait_ns(o_full, 0, abort_flag)) { set_error(a.err, ERR_WAIT_TMEM_FULL); *abort_flag = 1; ok = false; }
    if (ok) {
      tc_fence_after();
      const uint32_t o_tmem = tmem_base + lane_addr + 2 * FN;
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* dst = nullptr;
      if (row < valid_rows) {
        const int tk = row0_tok + tok_lo + row / G, head = kvh * G + row % G;
        dst = a.out + (size_t)tk * a.out_stride + (size_t)head * D;
      }
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(o_tmem + c * 32, r);
        tmem_ld_wait();
        if (dst != nullptr) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r[v * 8]) * inv, __uint_as_float(r[v * 8 + 1]) * inv);
            o.y = pack_bf16x2(__uint_as_float(r[v * 8 + 2]) * inv, __uint_as_float(r[v * 8 + 3]) * inv);
            o.z = pack_bf16x2(__uint_as_float(r[v * 8 + 4]) * inv, __uint_as_float(r[v * 8 + 5]) * inv);
            o.w = pack_bf16x2(__uint_as_float(r[v * 8 + 6]) * inv, __uint_as_float(r[v * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + v * 8) = o;
          }
        }
      }
    }
  }

  // ---------------- teardown ----------------
  pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0 && threadIdx.x == 0) {
    const uint64_t t0 = globaltimer_ns();       // let copies in flight land before the shared memory goes away
    while (globaltimer_ns() - t0 < 2000000ull) { __nanosleep(1000); }
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}


// ---- context attention over contiguous ragged K / V with unequal head dims (qk 192 / v 128) -------------------------------
// The prefill of a latent-attention (MLA) layer in its un-absorbed form: every head has its own keys (128 up-projected
// columns + 64 shared positional ones = 192) and values (128), freshly computed for the call, so K and V are plain
// ragged tensors [kv tokens][heads * dim], not pages. One CTA = (head, sequence, block of 128 query tokens); S = Q K^T
// over 192, O += P V over 128 columns, the same pipeline as above with 64-token KV tiles (256 TMEM columns).
// A query token i of a sequence with R new rows and L keys attends keys 0 .. L - R + i.
// Reference bar: kernel_index/trtllm_fmha_ctx_h192_v128.toml (a prebuilt blob there; no source counterpart).
struct CtxArgs {
  const __nv_bfloat16* q;       // [q tokens][q_stride], head h at column h * DQK
  __nv_bfloat16* out;           // [q tokens][out_stride], head h at column h * DV
  const int* cu_q;              // [seqs + 1]
  const int* cu_k;              // [seqs + 1]
  const int* work;
  const int* work_count;
  int* err;
  int q_stride, out_stride;
  float scale_log2;
};

// ST: stages of the K / V ring. 2: one CTA per SM (146 KB), the next tile's scores are issued before this tile's P V.
// 1: 106 KB, two CTAs per SM; the K and V halves have barriers of their own, so the next tile's K is loaded (and its
// scores issued) while this tile's softmax and P V still hold V: the one stage pipelines too.
template <int DQK, int DV, int FN, int ST>
struct CtxCfg {
  static constexpr int kQBytes = FM * DQK * 2;
  static constexpr int kPBytes = FM * FN * 2;
  static constexpr int kKBytes = FN * DQK * 2;
  static constexpr int kVBytes = FN * DV * 2;
  static constexpr int kStages = ST;
  static constexpr int kSlack = ST == 1 ? 768 : 1024;
  static constexpr int kSmem = kSlack + kQBytes + kPBytes + kStages * (kKBytes + kVBytes) + 256;
  static constexpr int kTmemCols = 2 * FN + DV <= 256 ? 256 : 512;
};

template <int DQK, int DV, int FN, int ST>
KERN_DEVICE void fmha_ctx_body(const CUtensorMap* k_map, const CUtensorMap* v_map, const CtxArgs& a) {
  using Cfg = CtxCfg<DQK, DV, FN, ST>;
  constexpr int kStages = Cfg::kStages;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  if ((int)(smem - smem_raw) > Cfg::kSlack) {             // uniform per CTA, before any barrier or allocation
    if (threadIdx.x == 0) set_error(a.err, ERR_BOUNDS);
    return;
  }
  uint8_t* q_s = smem;
  uint8_t* p_s = q_s + Cfg::kQBytes;
  uint8_t* kv_s = p_s + Cfg::kPBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(kv_s + kStages * (Cfg::kKBytes + Cfg::kVBytes));
  // K and V of a stage on barriers of their own, as in fmha_body: with one stage that alone lets the next tile's K load
  // (and Q K^T) run under this tile's softmax and P V
  uint64_t* k_full = bars;
  uint64_t* v_full = k_full + kStages;
  uint64_t* k_empty = v_full + kStages;
  uint64_t* v_empty = k_empty + kStages;
  uint64_t* s_full = v_empty + kStages;
  uint64_t* s_empty = s_full + 2;
  uint64_t* p_full = s_empty + 2;
  uint64_t* p_empty = p_full + 1;
  uint64_t* o_full = p_empty + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int y = blockIdx.y, head = blockIdx.x;
  if (y >= *a.work_count) return;                           // uniform per CTA, before any barrier or allocation
  if (*reinterpret_cast<volatile int*>(a.err) != 0) return;
  const int seq = a.work[2 * y], blk = a.work[2 * y + 1];
  const int row0_tok = a.cu_q[seq], R = a.cu_q[seq + 1] - row0_tok;
  const int k0 = a.cu_k[seq], L = a.cu_k[seq + 1] - k0;
  const int tok_lo = blk * FM;
  if (tok_lo >= R || L <= 0) return;
  const int valid_rows = min(FM, R - tok_lo);
  const int last_pos = min(L - 1, L - R + tok_lo + valid_rows - 1);
  if (last_pos < 0) return;                                 // more new rows than keys: these rows see nothing (left as they are)
  const int ntiles = last_pos / FN + 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&v_full[s], 1);
      mbar_init(&k_empty[s], 1); mbar_init(&v_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) { mbar_init(&s_full[b], 1); mbar_init(&s_empty[b], 128); }
    mbar_init(p_full, 128);
    mbar_init(p_empty, 1);
    mbar_init(o_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(k_map);
    tma_prefetch_desc(v_map);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();

  // Q tile -> shared memory, K-major with the 128-byte swizzle (DQK / 64 column blocks of [128 rows][128 bytes])
  for (int i = threadIdx.x; i < FM * (DQK / 8); i += blockDim.x) {
    const int r = i / (DQK / 8), c = i % (DQK / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < valid_rows)
      v = *reinterpret_cast<const uint4*>(a.q + (size_t)(row0_tok + tok_lo + r) * a.q_stride + (size_t)head * DQK + c * 8);
    const int cb = c >> 3, cc = c & 7;
    *reinterpret_cast<uint4*>(q_s + cb * (FM * 128) + r * 128 + ((cc ^ (r & 7)) << 4)) = v;
  }
  fence_proxy_async();
  __syncthreads();


  if (warp == 0) {
    // ---------------- producer: K (DQK / 64 boxes) and V (DV / 64 boxes) of every 64-token tile ----------------
    if (lane == 0) {
      auto load_half = [&](int t, int which) -> bool {
        const int stage = t % kStages;
        const uint32_t parity = ((t / kStages) & 1) ^ 1;
        if (!mbar_wait_ns(which ? &v_empty[stage] : &k_empty[stage], parity, abort_flag)) {
          set_error(a.err, ERR_WAIT_EMPTY);
          *abort_flag = 1;
          return false;
        }
        uint8_t* sk = kv_s + stage * (Cfg::kKBytes + Cfg::kVBytes);
        const int krow = k0 + t * FN;                 // rows past the sequence's end belong to the next one (or are out of
                                                      // range and read as zero): the causal limit masks them
        if (which == 0) {
          mbar_expect_tx(&k_full[stage], Cfg::kKBytes);
#pragma unroll
          for (int cb = 0; cb < DQK / 64; ++cb) tma_load_2d(sk + cb * (FN * 128), k_map, head * DQK + cb * 64, krow, &k_full[stage]);
        } else {
          uint8_t* sv = sk + Cfg::kKBytes;
          mbar_expect_tx(&v_full[stage], Cfg::kVBytes);
#pragma unroll
          for (int cb = 0; cb < DV / 64; ++cb) tma_load_2d(sv + cb * (FN * 128), v_map, head * DV + cb * 64, krow, &v_full[stage]);
        }
        return true;
      };
      // K(0), then K(t + 1) before V(t): the waits come in the order the MMAs complete
      bool ok = load_half(0, 0);
      for (int t = 0; t < ntiles && ok; ++t) {
        if (t + 1 < ntiles) ok = load_half(t + 1, 0);
        if (ok) ok = load_half(t, 1);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(FM, FN);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(FM, DV) | (1u << 16);      // B (= V) is MN-major
      const uint32_t o_tmem = tmem_base + 2 * FN;
      bool ok = true;
      auto issue_qk = [&](int j) {
        const int stage = j % kStages;
        if (!mbar_wait_ns(&k_full[stage], (j / kStages) & 1, abort_flag)) { set_error(a.err, ERR_WAIT_FULL); return false; }
        if (!mbar_wait_ns(&s_empty[j & 1], ((j >> 1) & 1) ^ 1, abort_flag)) { set_error(a.err, ERR_WAIT_TMEM_EMPTY); return false; }
        tc_fence_after();
        const uint32_t sq = smem_u32(q_s), sk = smem_u32(kv_s + stage * (Cfg::kKBytes + Cfg::kVBytes));
#pragma unroll
        for (int k = 0; k < DQK / 16; ++k)
          umma_bf16(tmem_base + (j & 1) * FN, umma_desc_sw128(sq + (k >> 2) * (FM * 128) + (k & 3) * 32),
                    umma_desc_sw128(sk + (k >> 2) * (FN * 128) + (k & 3) * 32), idesc_qk, k != 0);
        tc_commit(&s_full[j & 1]);
        tc_commit(&k_empty[stage]);         // the K half is free once these MMAs have read it
        return true;
      };
      auto issue_pv = [&](int j) {
        const int stage = j % kStages;
        if (!mbar_wait_ns(&v_full[stage], (j / kStages) & 1, abort_flag)) { set_error(a.err, ERR_WAIT_FULL); return false; }
        if (!mbar_wait_ns(p_full, j & 1, abort_flag)) { set_error(a.err, ERR_WAIT_FULL); return false; }
        tc_fence_after();
        const uint32_t sp = smem_u32(p_s), sv = smem_u32(kv_s + stage * (Cfg::kKBytes + Cfg::kVBytes) + Cfg::kKBytes);
#pragma unroll
        for (int k = 0; k < FN / 16; ++k)
          umma_bf16(o_tmem, umma_desc_sw128(sp + (k >> 2) * (FM * 128) + (k & 3) * 32),
                    umma_desc_sw128_mn(sv + k * 16 * 128, FN * 128), idesc_pv, (j | k) != 0);
        tc_commit(&v_empty[stage]);
        tc_commit(p_empty);
        if (j == ntiles - 1) tc_commit(o_full);
        return true;
      };
      ok = issue_qk(0);
      for (int j = 0; j < ntiles && ok; ++j) {
        // the next tile's scores first: they overlap this tile's softmax (with one stage too: its K half was free
        // as soon as this tile's Q K^T had read it)
        if (j + 1 < ntiles) ok = issue_qk(j + 1);
        if (ok) ok = issue_pv(j);
      }
      if (!ok) *abort_flag = 1;
    }
    __syncwarp();
  } else {
    // ---------------- softmax warps 2..5: one thread per query row (the scores of a 64-token tile stay in registers) ----------------
    static_assert(FN == 64, "the context kernel keeps a tile's scores in registers");
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const int pos = row < valid_rows ? (L - R + tok_lo + row) : -1;
    float m_ref = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < ntiles && ok; ++j) {
      if (!mbar_wait_ns(&s_full[j & 1], (j >> 1) & 1, abort_flag)) { set_error(a.err, ERR_WAIT_TMEM_FULL); *abort_flag = 1; ok = false; break; }
      tc_fence_after();
      const uint32_t s_tmem = tmem_base + lane_addr + (j & 1) * FN;
      const int tok0 = j * FN;
      const bool diag = tok0 + FN - 1 > pos;
      uint32_t keep[FN];
#pragma unroll
      for (int c = 0; c < FN / 32; ++c) tmem_ld_32x32(s_tmem + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&keep[c * 32]));
      tmem_ld_wait();
      if (diag) {         // the causal limit, once, on the scores themselves (a per-row branch: no warp-wide instruction inside)
#pragma unroll
        for (int i = 0; i < FN; ++i)
          if (tok0 + i > pos) keep[i] = 0xff800000u;        // -inf
      }
      float mx;
      {
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};        // four chains: a single one is 64 dependent steps
#pragma unroll
        for (int i = 0; i < FN; ++i) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(keep[i]));
        mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      }
      tc_fence_before();
      mbar_arrive(&s_empty[j & 1]);
      mx *= a.scale_log2;
      float alpha = 1.f;
      bool moved = false;
      if (mx > m_ref + 8.f) {
        alpha = m_ref == -INFINITY ? 0.f : exp2f(m_ref - mx);
        m_ref = mx;
        moved = true;
      }
      if (j > 0 && !mbar_wait_ns(p_empty, (j - 1) & 1, abort_flag)) { set_error(a.err, ERR_WAIT_EMPTY); *abort_flag = 1; ok = false; break; }
      tc_fence_after();
      if (__any_sync(0xffffffffu, moved && j > 0)) {        // warp-wide instructions: never under a per-row branch
        const uint32_t o_tmem = tmem_base + lane_addr + 2 * FN;
#pragma unroll 1
        for (int c = 0; c < DV / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(o_tmem + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st_32x32(o_tmem + c * 32, r);
        }
        tmem_st_wait();
      }
      l_run *= alpha;
      const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
      float sum = 0.f, sum_b = 0.f;
#pragma unroll
      for (int c = 0; c < FN / 32; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float p0 = exp2f(__uint_as_float(keep[c * 32 + 2 * i]) * a.scale_log2 - m_use);      // a masked score is -inf: 0
          const float p1 = exp2f(__uint_as_float(keep[c * 32 + 2 * i + 1]) * a.scale_log2 - m_use);
          if (i & 1) sum_b += p0 + p1; else sum += p0 + p1;
          pk[i] = pack_bf16x2(p0, p1);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int chunk = c * 4 + q, cb = chunk >> 3, cc = chunk & 7;
          *reinterpret_cast<uint4*>(p_s + cb * (FM * 128) + row * 128 + ((cc ^ (row & 7)) << 4)) =
              make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
        }
      }
      l_run += sum + sum_b;
      tc_fence_before();
      fence_proxy_async();
      mbar_arrive(p_full);
    }
    if (ok && !mbar_wait_ns(o_full, 0, abort_flag)) { set_error(a.err, ERR_WAIT_TMEM_FULL); *abort_flag = 1; ok = false; }
    if (__all_sync(0xffffffffu, ok)) {
      tc_fence_after();
      const uint32_t o_tmem = tmem_base + lane_addr + 2 * FN;
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* dst = row < valid_rows ? a.out + (size_t)(row0_tok + tok_lo + row) * a.out_stride + (size_t)head * DV : nullptr;
#pragma unroll 1
      for (int c = 0; c < DV / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(o_tmem + c * 32, r);
        tmem_ld_wait();
        if (dst != nullptr) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r[v * 8]) * inv, __uint_as_float(r[v * 8 + 1]) * inv);
            o.y = pack_bf16x2(__uint_as_float(r[v * 8 + 2]) * inv, __uint_as_float(r[v * 8 + 3]) * inv);
            o.z = pack_bf16x2(__uint_as_float(r[v * 8 + 4]) * inv, __uint_as_float(r[v * 8 + 5]) * inv);
            o.w = pack_bf16x2(__uint_as_float(r[v * 8 + 6]) * inv, __uint_as_float(r[v * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + v * 8) = o;
          }
        }
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0 && threadIdx.x == 0) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) { __nanosleep(1000); }
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}
}  // namespace kern

using namespace kern;

extern "C" __global__ void __launch_bounds__(192, 1)
    kern_attn_fmha_prefill_d128(const __grid_constant__ CUtensorMap kv_map, const __nv_bfloat16* q, __nv_bfloat16* out,
                                const int* block_table, const int* seq_lens, const int* cu_q, const int* work,
                                const int* work_count, int hq, int hk, int q_stride, int out_stride, int max_pages,
                                int page_size, int pool_pages, float scale_log2, int* err) {
  FmhaArgs a{q, out, block_table, seq_lens, cu_q, work, work_count, err, hq, hk, q_stride, out_stride, max_pages, page_size,
             pool_pages, scale_log2};
  fmha_body<128, 128>(&kv_map, a, (int)blockIdx.y);
}

extern "C" __global__ void __launch_bounds__(192, 2)
    kern_attn_fmha_prefill_d128_t64(const __grid_constant__ CUtensorMap kv_map, const __nv_bfloat16* q, __nv_bfloat16* out,
                                    const int* block_table, const int* seq_lens, const int* cu_q, const int* work,
                                    const int* work_count, int hq, int hk, int q_stride, int out_stride, int max_pages,
                                    int page_size, int pool_pages, float scale_log2, int* err) {
  FmhaArgs a{q, out, block_table, seq_lens, cu_q, work, work_count, err, hq, hk, q_stride, out_stride, max_pages, page_size,
             pool_pages, scale_log2};
  fmha_body<128, 64>(&kv_map, a, (int)blockIdx.y);
}

// Both lists of a ragged call in one launch: the CTAs of this kernel (list p: prompt chunks, 64-token KV tiles) and of
// the token-parallel mma.sync kernel (list d: decode rows, a two-stage ring) alternate in launch order while both
// lists last. Either kind takes half an SM (113 KB / 84 KB of shared memory, 256 TMEM columns for this one, none for
// the other), so a prompt tile's tensor-core work and softmax share the SM with a decode sequence's KV stream.
// block = 192: a decode CTA retires its sixth warp at once. grid = (hk, at least count_p + count_d).
extern "C" __global__ void __launch_bounds__(192, 2)
    kern_attn_ragged_fmha_d128(const __grid_constant__ CUtensorMap kv_map, const __nv_bfloat16* q, __nv_bfloat16* out,
                               const int* block_table, const int* seq_lens, const int* cu_q, const int* work_p,
                               const int* count_p, const int* work_d, const int* count_d, int hq, int hk, int q_stride,
                               int out_stride, int max_pages, int page_size, int pool_pages, float scale_log2, int* err) {
  const int np = *count_p, nd = *count_d, m = np < nd ? np : nd;
  const int y = blockIdx.y;
  if (y >= np + nd) return;
  const bool is_p = y < 2 * m ? !(y & 1) : np > nd;
  const int idx = y < 2 * m ? (y >> 1) : y - m;
  if (is_p) {
    FmhaArgs a{q, out, block_table, seq_lens, cu_q, work_p, count_p, err, hq, hk, q_stride, out_stride, max_pages, page_size,
               pool_pages, scale_log2};
    fmha_body<128, 64>(&kv_map, a, idx);
  } else {
    if (threadIdx.x >= 160) return;          // the token-parallel kernel is written for five warps
    AttnArgs a{q, out, nullptr, nullptr, block_table, seq_lens, cu_q, work_d, count_d, err, 0x7fffffff, hq, hk, q_stride,
               out_stride, max_pages, page_size, 1, 1, pool_pages, scale_log2};
    attn_body<128, false, 2>(&kv_map, a, idx);
  }
}

// grid = (heads, work items), block 192, dynamic shared memory CtxCfg<192, 128, 64, ST>::kSmem
#define KERN_FMHA_CTX_ENTRY(name, ST, PER_SM)                                                                                  \
  extern "C" __global__ void __launch_bounds__(192, PER_SM)                                                                    \
      name(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map, const __nv_bfloat16* q,        \
           __nv_bfloat16* out, const int* cu_q, const int* cu_k, const int* work, const int* work_count, int q_stride,          \
           int out_stride, float scale_log2, int* err) {                                                                       \
    CtxArgs a{q, out, cu_q, cu_k, work, work_count, err, q_stride, out_stride, scale_log2};                                     \
    fmha_ctx_body<192, 128, 64, ST>(&k_map, &v_map, a);                                                                        \
  }

KERN_FMHA_CTX_ENTRY(kern_attn_fmha_ctx_qk192_v128, 2, 1)
KERN_FMHA_CTX_ENTRY(kern_attn_fmha_ctx_qk192_v128_x2, 1, 2)
