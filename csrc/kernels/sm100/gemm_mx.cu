// Block-scaled GEMM on the 5th-generation tensor cores: C[M, N] (bf16) = (A ⊙ SFA) · (W ⊙ SFW)^T with one UE8M0
// (power-of-two) scale per 32 elements along K — the OCP microscaling formats:
//   A  : MXFP8, e4m3 bytes [M, K]
//   W  : MXFP8 e4m3 bytes [N, K], or MXFP4 e2m1 nibbles [N, K/2] (element 2i in the low nibble of byte i)
// `tcgen05.mma.kind::mxf8f6f4.block_scale` multiplies the scales in hardware: the scale factors of a stage are copied
// from shared memory into TMEM (`tcgen05.cp`) by the thread that issues the MMAs, ahead of them, and each K = 32
// instruction picks its byte through the instruction descriptor. The rest is the dense pipeline: a TMA producer warp
// filling a ring of 128-byte-swizzled stages (K = 128 per stage), one elected MMA thread, four epilogue warps reading
// the f32 accumulator out of TMEM, two accumulators so the epilogue of tile i overlaps the main loop of tile i + 1.
// MXFP4 weights travel from HBM as packed nibbles (half the bytes of fp8: what bounds a decode step) and are unpacked
// by the TMA unit itself (tensor-map type 16U4_ALIGN16B: 16 nibbles land in the low half of a 16-byte chunk), so in
// shared memory they look like an 8-bit operand to the instruction.
//
// Scale-factor layout in global memory ("atoms"): for a matrix of R rows and K/32 blocks, atom (R/128, kb/4) is 512
// bytes at ((r / 128) * ceil(K / 128) + kb / 4) * 512, and inside it the scale of row r, block kb sits at
//   (r % 32) * 16 + ((r / 32) % 4) * 4 + kb % 4.
// That is the order `tcgen05.cp ... 32x128b.warpx4` wants: one bulk copy brings an atom into shared memory and one
// tcgen05.cp puts it in four TMEM columns (lane r % 32 of every quadrant, column (r / 32) % 4, byte kb % 4).
//
// Serves `extern:cublaslt_mxfp8_tn` (reference: crates/kern-runtime/src/cublas.rs:401-505, VEC32_UE8M0 at :459) and, in
// the grouped form over the MoE planner's tile table, the routed expert GEMMs the reference takes from prebuilt blobs
// (kernel_index/trtllm_bmm_mxe4m3_mxe2m1_mxe4m3.toml, trtllm_bmm_bf16_mxe2m1_mxe4m3.toml).
// Every mbarrier wait is bounded; a wait that runs out sets *err and the CTA unwinds (TMEM freed).
#include "common.cuh"

#include <cuda_fp8.h>

namespace kern {

constexpr int MX_BM = 128;
constexpr int MX_BK = 128;            // elements of K per stage = one 128-byte swizzle row of 8-bit (or unpacked 4-bit) data
constexpr int MX_SF_ATOM = 512;       // bytes of one 128-row x 4-block scale atom

template <int BN>
struct MxCfg {
  static constexpr int kBytesA = MX_BM * MX_BK;
  static constexpr int kBytesB = BN * MX_BK;
  static constexpr int kBytesSfa = MX_SF_ATOM;
  static constexpr int kBytesSfb = (BN / 128) * MX_SF_ATOM;
  static constexpr int kBytesSf = BN == 256 ? 2048 : 1024;           // room for the scale atoms, keeping A and B 1024-aligned
  static constexpr int kStageBytes = kBytesA + kBytesB + kBytesSf;
  static constexpr int kStages = BN == 256 ? 4 : 6;
  static constexpr int kAccs = BN == 256 ? 1 : 2;
  static constexpr int kSfCols = 4 + BN / 32;                       // TMEM columns of the scales of one stage
  static constexpr int kTmemCols = 512;
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + 256;
};

// Instruction descriptor of kind::mxf8f6f4.block_scale: A/B formats (e4m3 = 0, e2m1 = 5), both K-major, UE8M0 scales,
// N >> 3 at bit 17, M >> 4 at bit 24; which of a column's four scale bytes each operand uses at bits 29 (A) and 4 (B).
KERN_DEVICE constexpr uint32_t mx_idesc(int m, int n, int b_format) {
  return ((uint32_t)0 << 7) | ((uint32_t)b_format << 10) | ((uint32_t)(n >> 3) << 17) | (1u << 23) | ((uint32_t)(m >> 4) << 24);
}

KERN_DEVICE void umma_mx(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem,
                         uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
      : "memory");
}

// 32 rows x 16 bytes of shared memory (rows 16 bytes apart: four 8-row core matrices 128 bytes apart, no swizzle) into
// four TMEM columns, the same 32 lanes in every quadrant.
KERN_DEVICE uint64_t sf_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)(16 >> 4) << 16;                 // leading byte offset (one core matrix along K: unused)
  d |= (uint64_t)(128 >> 4) << 32;                // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                         // descriptor version
  return d;                                       // layout type 0: no swizzle
}
KERN_DEVICE void tmem_cp_sf(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}

// GROUPED: M tiles come from the MoE planner's table of int4 {expert, first row (a multiple of 128), rows, -}; W and its
// scales are per expert (3-D weight map [K, N, experts]; scale atoms of expert e at sfw + e * sfw_expert_bytes).
// A tile of packed nibbles completes the stage's barrier with the bytes read from global memory (two elements per
// byte), not with the 128 bytes per row it occupies in shared memory.
//
// EPI 0: bf16 store. EPI 1 (the first expert GEMM): W's rows come in groups of 128 = 64 gate rows then the matching 64 up
// rows (interleaved when the weights are prepared), so accumulator columns [128 g, 128 g + 64) are gate and the next 64
// the matching up columns; the epilogue computes silu(gate) * up and writes it as MXFP8 — an epilogue thread holds a
// whole 32-element block of its row, so the block's scale needs no exchange between threads — with the scales in the
// atom layout, ready to be the A operand of the second expert GEMM. C is then e4m3 bytes [rows, N / 2].
//
// Expert parallel over sharded tokens (both forms GROUPED, over the aligned plan of moe.cu::kern_moe_plan_ep):
//   EP == 1, dispatch fused into the first expert GEMM: every home rank quantises its activations once (MXFP8 bytes and
//     row-major scales, kern_quant_mxfp8_rows, both buffers exported); four extra warps pull row r of the expert-sorted
//     operand (token src_tok[r]) out of its home rank — the K e4m3 bytes into `xq`, the K / 32 scale bytes word by
//     word into the row's place in the local scale atoms — and count the row into its 128-row block's arrival counter.
//     The producer waits (bounded) for a block's BM arrivals before the first load of a tile; counters only grow (every
//     launch adds BM to each), so graphs replay. Half the bytes of the bf16 dispatch cross NVLink.
//   EPI == 2, combine fused into the second expert GEMM: row r of the bf16 result goes from TMEM, through a
//     shared-memory staging block so that every peer store covers a 128-byte line, into slot (token, choice) of the
//     return buffer on the token's home rank; the last CTA to finish publishes this rank's epoch into every rank's
//     `done` words (moe.cu::kern_ep_finalize waits for them and forms the weighted sum).
struct MxEpArgs {
  const unsigned long long* x_peers = nullptr;    // dispatch: every rank's quantised activations [rows_per_rank, K] e4m3
  const unsigned long long* sf_peers = nullptr;   //           and their scales [rows_per_rank, K / 32], row-major
  uint8_t* xq = nullptr;                          //           this rank's expert-sorted rows (the A operand)
  uint8_t* sfa = nullptr;                         //           and their scale atoms
  uint32_t* flags = nullptr;                      //           [max_blocks] rows arrived per 128-row block
  uint32_t* epochs = nullptr;                     //           [grid] launches seen by each CTA
  int max_blocks = 0;
  const int* src_tok = nullptr;                   // both: global token of each expert-sorted row, -1 for padding
  const int* row_choice = nullptr;                // combine: which of its token's k choices the row is
  const unsigned long long* ret_peers = nullptr;  //          every rank's return buffer [rows_per_rank, k, N] bf16
  const unsigned long long* done_peers = nullptr; //          every rank's done words [nranks]
  uint32_t* state = nullptr;                      //          {CTAs finished, epoch}
  int rows_per_rank = 1, rank = 0, nranks = 1, k = 1;
};
constexpr int kMxGatherWarps = 4;
constexpr int kMxWindow = 8;                      // 128-row blocks per window of the dispatch form's tile order
constexpr int kMxSlotStage = 4 * (32 * 144 + 256);   // shared memory of the combine form's row staging

template <int BN, bool B_FP4, bool GROUPED, int EPI = 0, int EP = 0>
__device__ __forceinline__ void mx_gemm_body(const CUtensorMap* tma_a, const CUtensorMap* tma_b, const uint8_t* sfa,
                                             const uint8_t* sfw, void* Cv, int M, int N, int K, int ldc, int* err,
                                             const int* tile_table, const int* tile_count, long long sfw_expert_bytes,
                                             uint8_t* sf_out = nullptr, MxEpArgs ep = MxEpArgs()) {
  static_assert((EP == 0 && EPI != 2) || GROUPED, "the expert-parallel forms are routed GEMMs");
  __nv_bfloat16* C = reinterpret_cast<__nv_bfloat16*>(Cv);
  using Cfg = MxCfg<BN>;
  constexpr int kStages = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * Cfg::kStageBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tfull_bar = empty_bar + kStages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_n = (N + BN - 1) / BN;
  const int num_kb = (K + MX_BK - 1) / MX_BK;     // = scale atoms along K

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull_bar[a], 1); mbar_init(&tempty_bar[a], 4); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) { tma_prefetch_desc(tma_a); tma_prefetch_desc(tma_b); }
  pdl_wait();
  const int num_m = GROUPED ? *tile_count : (M + MX_BM - 1) / MX_BM;
  const int num_tiles = num_m * num_n;
  uint32_t ep_want = 0;
  if constexpr (EP == 1) {
    ep_want = (ep.epochs[blockIdx.x] + 1u) * (uint32_t)MX_BM;
    __syncthreads();      // every thread has read this CTA's launch count before the gather warps write the next one
  }
  auto tile_of = [&](int t, int& row0, int& row_end, int& n_blk, int& expert) {
    int mt = t % num_m;
    n_blk = t / num_m;
    if constexpr (EP == 1) {
      // blocks in the order their rows arrive, kMxWindow at a time with the row blocks fastest inside a window: the
      // first wave needs only the first few blocks, and CTAs that run together share W tiles through L2
      const int per_win = kMxWindow * num_n;
      const int w = t / per_win, r = t - w * per_win;
      const int m0 = w * kMxWindow, wm = min(kMxWindow, num_m - m0);
      mt = m0 + r % wm;
      n_blk = r / wm;
    }
    if constexpr (GROUPED) {
      const int4 e = reinterpret_cast<const int4*>(tile_table)[mt];
      expert = e.x; row0 = e.y; row_end = min(M, e.y + e.z);
    } else {
      expert = 0; row0 = mt * MX_BM; row_end = M;
    }
  };

  if (warp == 0) {
    // ---------------- producer: TMA tiles + bulk copies of the scale atoms ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int row0, row_end, n_blk, expert;
        tile_of(t, row0, row_end, n_blk, expert);
        if constexpr (EP == 1) {
          const int blk = row0 / MX_BM;
          bool here = false;
          for (uint32_t i = 0; i < (1u << 22) && !here; ++i) {
            here = ld_acquire_sys(ep.flags + blk) >= ep_want;
            if (!here) { if ((i & 0xff) == 0xff && *abort_flag != 0) break; __nanosleep(100); }
          }
          if (!here) {
            set_error(err, ERR_WAIT_PEER + ep.nranks);
            *abort_flag = 1;
            break;
          }
          asm volatile("fence.proxy.async;" ::: "memory");   // rows and scales were written by ordinary stores; bulk copies read them
        }
        const uint8_t* sfa_row = sfa + (size_t)(row0 / MX_BM) * num_kb * MX_SF_ATOM;
        const uint8_t* sfw_base = sfw + (GROUPED ? (size_t)expert * sfw_expert_bytes : 0);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
            set_error(err, ERR_WAIT_EMPTY);
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kBytesA;
          uint8_t* ssfa = sb + Cfg::kBytesB;
          uint8_t* ssfb = ssfa + Cfg::kBytesSfa;
          mbar_expect_tx(&full_bar[stage], Cfg::kBytesA + (B_FP4 ? Cfg::kBytesB / 2 : Cfg::kBytesB) + Cfg::kBytesSfa + Cfg::kBytesSfb);
          tma_load_2d(sa, tma_a, kb * MX_BK, row0, &full_bar[stage]);
          if constexpr (GROUPED) tma_load_3d(sb, tma_b, kb * MX_BK, n_blk * BN, expert, &full_bar[stage]);
          else tma_load_2d(sb, tma_b, kb * MX_BK, n_blk * BN, &full_bar[stage]);
          bulk_load_1d(ssfa, sfa_row + (size_t)kb * MX_SF_ATOM, Cfg::kBytesSfa, &full_bar[stage]);
#pragma unroll
          for (int j = 0; j < BN / 128; ++j)
            bulk_load_1d(ssfb + j * MX_SF_ATOM, sfw_base + ((size_t)(n_blk * (BN / 128) + j) * num_kb + kb) * MX_SF_ATOM,
                         MX_SF_ATOM, &full_bar[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc0 = mx_idesc(MX_BM, BN, B_FP4 ? 5 : 0);
      const uint32_t sf_tmem = tmem_base + Cfg::kAccs * BN;          // scale columns sit behind the accumulators
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag)) {
          set_error(err, ERR_WAIT_TMEM_EMPTY);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
            set_error(err, ERR_WAIT_FULL);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t sb = sa + Cfg::kBytesA;
          const uint32_t ssfa = sb + Cfg::kBytesB;
          const uint32_t ssfb = ssfa + Cfg::kBytesSfa;
          // scales of this stage into TMEM, in issue order ahead of the MMAs that read them
          tmem_cp_sf(sf_tmem, sf_desc(ssfa));
#pragma unroll
          for (int j = 0; j < BN / 128; ++j) tmem_cp_sf(sf_tmem + 4 + 4 * j, sf_desc(ssfb + j * MX_SF_ATOM));
#pragma unroll
          for (int k = 0; k < MX_BK / 32; ++k) {
            const uint32_t idesc = idesc0 | ((uint32_t)k << 29) | ((uint32_t)k << 4);   // scale byte k of A and of B
            umma_mx(d_tmem, umma_desc_sw128(sa + k * 32), umma_desc_sw128(sb + k * 32), idesc, sf_tmem, sf_tmem + 4,
                    (kb | k) != 0);
          }
          tc_commit(&empty_bar[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit(&tfull_bar[acc]);
        if (++acc == Cfg::kAccs) { acc = 0; acc_phase ^= 1; }
      }
    }
    __syncwarp();
  } else if (warp >= 6) {
    // ---------------- gather warps 6..9 (dispatch form): a warp per expert-sorted row ----------------
    if constexpr (EP == 1) {
      const int gw = blockIdx.x * kMxGatherWarps + (warp - 6), GW = gridDim.x * kMxGatherWarps;
      const int row_vecs = K / 16, sf_words = K / 128, total_rows = num_m * MX_BM;
      for (int b = num_m + gw * 32 + lane; b < ep.max_blocks; b += GW * 32) atomicAdd(ep.flags + b, (uint32_t)MX_BM);   // unused this launch
      auto ld8 = [&](const uint8_t* src, int v0, uint4 (&x)[8]) {
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const int v = v0 + q * 32;
          if (v < row_vecs)
            asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(x[q].x), "=r"(x[q].y), "=r"(x[q].z), "=r"(x[q].w) : "l"(src + (size_t)v * 16));
        }
      };
      for (int r = gw; r < total_rows && *abort_flag == 0; r += GW) {
        const int tok = ep.src_tok[r];
        if (tok >= 0) {
          const int home = tok / ep.rows_per_rank, lr = tok % ep.rows_per_rank;
          const uint8_t* src = reinterpret_cast<const uint8_t*>(ep.x_peers[home]) + (size_t)lr * K;
          const uint32_t* ssrc = reinterpret_cast<const uint32_t*>(ep.sf_peers[home]) + (size_t)lr * sf_words;
          uint32_t sw[4];
#pragma unroll
          for (int q = 0; q < 4; ++q)
            if (lane + q * 32 < sf_words)
              asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(sw[q]) : "l"(ssrc + lane + q * 32));
          uint4* dst = reinterpret_cast<uint4*>(ep.xq + (size_t)r * K);
          uint4 xa[8], xb[8];
          const bool ok_row = KERN_CHECK(src, (size_t)K, SITE_EP_PULL) && KERN_CHECK(dst, (size_t)K, SITE_MOE_GATHER);
          if (ok_row) ld8(src, lane, xa);
          for (int v0 = lane; ok_row && v0 < row_vecs; v0 += 256) {
            if (v0 + 256 < row_vecs) ld8(src, v0 + 256, xb);
#pragma unroll
            for (int q = 0; q < 8; ++q)
              if (v0 + q * 32 < row_vecs) dst[v0 + q * 32] = xa[q];
#pragma unroll
            for (int q = 0; q < 8; ++q) xa[q] = xb[q];
          }
          // the row's four scale bytes of K block w sit in atom (r / 128, w)
          uint8_t* sdst = ep.sfa + (size_t)(r / MX_BM) * num_kb * MX_SF_ATOM + (r % 32) * 16 + ((r / 32) % 4) * 4;
#pragma unroll
          for (int q = 0; q < 4; ++q)
            if (lane + q * 32 < sf_words) *reinterpret_cast<uint32_t*>(sdst + (size_t)(lane + q * 32) * MX_SF_ATOM) = sw[q];
          for (int w = lane + 128; w < sf_words; w += 32) {      // K beyond 16384
            uint32_t v;
            asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(ssrc + w));
            *reinterpret_cast<uint32_t*>(sdst + (size_t)w * MX_SF_ATOM) = v;
          }
          __threadfence();
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        __syncwarp();
        if (lane == 0) atomicAdd(ep.flags + (r >> 7), 1u);
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kMxGatherWarps * 32) : "memory");
      if (threadIdx.x == 192) ep.epochs[blockIdx.x] = ep_want / MX_BM;
    }
  } else {
    // ---------------- epilogue warps 2..5 ----------------
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int row0, row_end, n_blk, expert;
      tile_of(t, row0, row_end, n_blk, expert);
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag)) {
        set_error(err, ERR_WAIT_TMEM_FULL);
        *abort_flag = 1;
        break;
      }
      tc_fence_after();
      const int row = row0 + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
      if constexpr (EPI == 1) {
        uint8_t* Q = reinterpret_cast<uint8_t*>(Cv);
        const int out_atoms = (N / 2 + MX_BK - 1) / MX_BK;             // scale atoms along the output's K
#pragma unroll 1
        for (int gc = 0; gc < BN / 64; ++gc) {                          // 32 output columns at a time
          const int g = gc >> 1, c = gc & 1;
          uint32_t gate[32], up[32];
          tmem_ld_32x32(t_row + g * 128 + c * 32, gate);
          tmem_ld_32x32(t_row + g * 128 + 64 + c * 32, up);
          tmem_ld_wait();
          const int col = n_blk * (BN / 2) + g * 64 + c * 32;           // output column of the block
          if (row < row_end && col < N / 2) {
            float a[32];
            float amax = 0.f;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              a[j] = silu(__uint_as_float(gate[j])) * __uint_as_float(up[j]);
              amax = fmaxf(amax, fabsf(a[j]));
            }
            int e = 0;
            if (amax > 0.f) {
              int ex;
              const float mant = frexpf(amax, &ex);
              e = mant <= 0.875f ? ex - 9 : ex - 8;
              e = max(-127, min(127, e));
            }
            const float inv = exp2f((float)-e);
            uint32_t w[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              uint32_t b = 0;
#pragma unroll
              for (int q = 0; q < 4; ++q)
                b |= (uint32_t)__nv_cvt_float_to_fp8(a[j * 4 + q] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * q);
              w[j] = b;
            }
            uint4* dst = reinterpret_cast<uint4*>(Q + (size_t)row * ldc + col);
            dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
            dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
            const int kb = col / 32;
            sf_out[((size_t)(row / 128) * out_atoms + kb / 4) * MX_SF_ATOM + (row % 32) * 16 + ((row / 32) % 4) * 4 + kb % 4] =
                (uint8_t)(e + 127);
          }
        }
      } else if constexpr (EPI == 2) {
        // A lane first works out where its own row lands (once per tile); then, 64 columns at a time, the warp parks its
        // 32 x 64 block in shared memory and writes it out four rows per instruction, eight lanes per row.
        static_assert(Cfg::kSmemBytes + 512 + kMxSlotStage <= 232448, "stages plus the row staging fit a CTA's shared memory");
        uint8_t* stage = smem + kStages * Cfg::kStageBytes + 512 + quarter * (32 * 144 + 256);
        unsigned long long* rowptr = reinterpret_cast<unsigned long long*>(stage + 32 * 144);
        {
          unsigned long long dst = 0;
          if (row < row_end) {
            const int tok = ep.src_tok[row];
            if (tok >= 0)
              dst = ep.ret_peers[tok / ep.rows_per_rank] +
                    2ull * (((size_t)(tok % ep.rows_per_rank) * ep.k + ep.row_choice[row]) * (size_t)N);
            if (dst != 0 && !KERN_CHECK(reinterpret_cast<const void*>(dst), (size_t)N * 2, SITE_EP_SLOT)) dst = 0;
          }
          rowptr[lane] = dst;
        }
        __syncwarp();
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(t_row + c * 64, r0);
          tmem_ld_32x32(t_row + c * 64 + 32, r1);
          tmem_ld_wait();
          uint4* mine = reinterpret_cast<uint4*>(stage + lane * 144);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r0[v * 8]), __uint_as_float(r0[v * 8 + 1]));
            o.y = pack_bf16x2(__uint_as_float(r0[v * 8 + 2]), __uint_as_float(r0[v * 8 + 3]));
            o.z = pack_bf16x2(__uint_as_float(r0[v * 8 + 4]), __uint_as_float(r0[v * 8 + 5]));
            o.w = pack_bf16x2(__uint_as_float(r0[v * 8 + 6]), __uint_as_float(r0[v * 8 + 7]));
            mine[v] = o;
            o.x = pack_bf16x2(__uint_as_float(r1[v * 8]), __uint_as_float(r1[v * 8 + 1]));
            o.y = pack_bf16x2(__uint_as_float(r1[v * 8 + 2]), __uint_as_float(r1[v * 8 + 3]));
            o.z = pack_bf16x2(__uint_as_float(r1[v * 8 + 4]), __uint_as_float(r1[v * 8 + 5]));
            o.w = pack_bf16x2(__uint_as_float(r1[v * 8 + 6]), __uint_as_float(r1[v * 8 + 7]));
            mine[4 + v] = o;
          }
          __syncwarp();
          const int col = n_blk * BN + c * 64 + (lane & 7) * 8;
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int rr = it * 4 + (lane >> 3);
            const unsigned long long dst = rowptr[rr];
            if (dst != 0 && col < N) {
              const uint4 val = *reinterpret_cast<const uint4*>(stage + rr * 144 + (lane & 7) * 16);
              *reinterpret_cast<uint4*>(dst + 2ull * col) = val;
            }
          }
          __syncwarp();
        }
      } else {
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col = n_blk * BN + c * 32;
        if (row < row_end) {
          __nv_bfloat16* out = C + (size_t)row * ldc + col;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            if (col + v * 8 < N) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r[v * 8]), __uint_as_float(r[v * 8 + 1]));
              o.y = pack_bf16x2(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
              o.z = pack_bf16x2(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
              o.w = pack_bf16x2(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
              *reinterpret_cast<uint4*>(out + v * 8) = o;
            }
          }
        }
      }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      if (++acc == Cfg::kAccs) { acc = 0; acc_phase ^= 1; }
    }
  }

  // ---------------- teardown ----------------
  if constexpr (EPI == 2) __threadfence_system();   // the pushed rows are on their way before the kernel is done
  pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  if constexpr (EPI == 2) {
    // the last CTA to get here publishes this rank's epoch: every store of this launch is ordered before it
    if (threadIdx.x == 0) {
      __threadfence_system();
      if (atomicAdd(ep.state, 1u) == gridDim.x - 1) {
        ep.state[0] = 0;
        const uint32_t e = ep.state[1] + 1;
        ep.state[1] = e;
        __threadfence_system();
        for (int r = 0; r < ep.nranks; ++r) st_release_sys(reinterpret_cast<uint32_t*>(ep.done_peers[r]) + ep.rank, e);
      }
    }
  }
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

}  // namespace kern

using namespace kern;

#define KERN_MX_GEMM_ENTRY(name, BN, FP4)                                                                          \
  extern "C" __global__ void __launch_bounds__(192, 1)                                                             \
      name(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const uint8_t* sfa,   \
           const uint8_t* sfw, __nv_bfloat16* C, int M, int N, int K, int ldc, int* err) {                           \
    kern::mx_gemm_body<BN, FP4, false>(&tma_a, &tma_b, sfa, sfw, C, M, N, K, ldc, err, nullptr, nullptr, 0);         \
  }
#define KERN_MX_GROUPED_ENTRY(name, BN, FP4, EPI)                                                                  \
  extern "C" __global__ void __launch_bounds__(192, 1)                                                             \
      name(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const uint8_t* sfa,   \
           const uint8_t* sfw, void* C, int M, int N, int K, int ldc, int* err, const int* tile_table,               \
           const int* tile_count, long long sfw_expert_bytes, uint8_t* sf_out) {                                   \
    kern::mx_gemm_body<BN, FP4, true, EPI>(&tma_a, &tma_b, sfa, sfw, C, M, N, K, ldc, err, tile_table, tile_count,   \
                                           sfw_expert_bytes, sf_out);                                              \
  }

KERN_MX_GEMM_ENTRY(kern_gemm_mxfp8_tn_n128, 128, false)
KERN_MX_GEMM_ENTRY(kern_gemm_mxfp8_tn_n256, 256, false)
KERN_MX_GEMM_ENTRY(kern_gemm_mxfp8_mxfp4_tn_n128, 128, true)
KERN_MX_GEMM_ENTRY(kern_gemm_mxfp8_mxfp4_tn_n256, 256, true)
KERN_MX_GROUPED_ENTRY(kern_moe_gemm_mxfp8_mxfp4_n128, 128, true, 0)
KERN_MX_GROUPED_ENTRY(kern_moe_gemm_mxfp8_mxfp4_n256, 256, true, 0)
KERN_MX_GROUPED_ENTRY(kern_moe_gemm_mxfp8_mxfp4_swiglu_mxfp8_n128, 128, true, 1)
KERN_MX_GROUPED_ENTRY(kern_moe_gemm_mxfp8_mxfp4_swiglu_mxfp8_n256, 256, true, 1)

// The expert-parallel pair (dispatch inside the first routed GEMM, combine inside the second).
#define KERN_EP_MX_FC1_ENTRY(name, BN)                                                                             \
  extern "C" __global__ void __launch_bounds__(320, 1)                                                             \
      name(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, uint8_t* sfa,         \
           const uint8_t* sfw, void* C, int M, int N, int K, int ldc, int* err, const int* tile_table,               \
           const int* tile_count, long long sfw_expert_bytes, uint8_t* sf_out, const unsigned long long* x_peers,   \
           const unsigned long long* sf_peers, uint8_t* xq, const int* src_tok, uint32_t* flags,                     \
           uint32_t* cta_epochs, int rows_per_rank, int max_blocks, int nranks) {                                  \
    kern::MxEpArgs ep;                                                                                             \
    ep.x_peers = x_peers; ep.sf_peers = sf_peers; ep.xq = xq; ep.sfa = sfa; ep.flags = flags; ep.epochs = cta_epochs; \
    ep.max_blocks = max_blocks; ep.src_tok = src_tok; ep.rows_per_rank = rows_per_rank; ep.nranks = nranks;        \
    if (*tile_count > max_blocks || (K % 128) != 0) { /* every 128-row block needs its counter */                  \
      if (threadIdx.x == 0 && blockIdx.x == 0) kern::set_error(err, kern::ERR_BOUNDS);                             \
      return;                                                                                                      \
    }                                                                                                              \
    kern::mx_gemm_body<BN, true, true, 1, 1>(&tma_a, &tma_b, sfa, sfw, C, M, N, K, ldc, err, tile_table, tile_count,  \
                                             sfw_expert_bytes, sf_out, ep);                                        \
  }
#define KERN_EP_MX_FC2_ENTRY(name, BN)                                                                             \
  extern "C" __global__ void __launch_bounds__(192, 1)                                                             \
      name(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const uint8_t* sfa,   \
           const uint8_t* sfw, int M, int N, int K, int* err, const int* tile_table, const int* tile_count,          \
           long long sfw_expert_bytes, const unsigned long long* ret_peers, const int* src_tok,                     \
           const int* row_choice, uint32_t* state, const unsigned long long* done_peers, int rows_per_rank, int k,  \
           int rank, int nranks) {                                                                                 \
    kern::MxEpArgs ep;                                                                                             \
    ep.ret_peers = ret_peers; ep.src_tok = src_tok; ep.row_choice = row_choice; ep.state = state;                  \
    ep.done_peers = done_peers; ep.rows_per_rank = rows_per_rank; ep.k = k; ep.rank = rank; ep.nranks = nranks;    \
    kern::mx_gemm_body<BN, true, true, 2>(&tma_a, &tma_b, sfa, sfw, nullptr, M, N, K, N, err, tile_table, tile_count, \
                                          sfw_expert_bytes, nullptr, ep);                                          \
  }
KERN_EP_MX_FC1_ENTRY(kern_ep_fc1_mxfp8_mxfp4_swiglu_mxfp8_n128, 128)
KERN_EP_MX_FC1_ENTRY(kern_ep_fc1_mxfp8_mxfp4_swiglu_mxfp8_n256, 256)
KERN_EP_MX_FC2_ENTRY(kern_ep_fc2_mxfp8_mxfp4_combine_n128, 128)
KERN_EP_MX_FC2_ENTRY(kern_ep_fc2_mxfp8_mxfp4_combine_n256, 256)

// ---- quantiser: bf16 rows -> MXFP8 (e4m3 + one UE8M0 scale per 32 elements, scales in the atom layout) -------------
// scale = 2^ceil(log2(amax / 448)) (the smallest power of two that brings the block into e4m3's range), clamped to the
// UE8M0 range; an all-zero block gets scale 1. One warp per (row, 32-element block): lane = element.
// grid any, block 256; K a multiple of 32. Rows >= M of a partly filled atom are left untouched.
extern "C" __global__ void kern_quant_mxfp8(const __nv_bfloat16* x, uint8_t* q, uint8_t* sf, int M, int K, int ldx) {
  const int lane = threadIdx.x & 31;
  const long long blocks_per_row = K / 32;
  const long long total = (long long)M * blocks_per_row;
  const int katoms = (K + MX_BK - 1) / MX_BK;
  for (long long b = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); b < total; b += (long long)gridDim.x * 8) {
    const int row = (int)(b / blocks_per_row), kb = (int)(b % blocks_per_row);
    const float v = __bfloat162float(x[(size_t)row * ldx + kb * 32 + lane]);
    const float amax = warp_max(fabsf(v));
    int e = 0;                                                  // scale = 2^e, the least power of two with amax <= 448 * 2^e
    if (amax > 0.f) {
      int ex;
      const float mant = frexpf(amax, &ex);                     // amax = mant * 2^ex, mant in [0.5, 1); 448 = 0.875 * 2^9
      e = mant <= 0.875f ? ex - 9 : ex - 8;
      e = max(-127, min(127, e));
    }
    const float inv = exp2f((float)-e);
    q[(size_t)row * K + kb * 32 + lane] = (uint8_t)__nv_cvt_float_to_fp8(v * inv, __NV_SATFINITE, __NV_E4M3);
    if (lane == 0)
      sf[((size_t)(row / 128) * katoms + kb / 4) * MX_SF_ATOM + (row % 32) * 16 + ((row / 32) % 4) * 4 + kb % 4] =
          (uint8_t)(e + 127);
  }
}

// The same quantiser with the scales row-major ([M, K / 32] bytes): what a home rank exports for the fused expert-parallel
// dispatch — a peer pulls a row's K / 32 scale bytes as K / 128 words and drops each into its atom. Four threads share a
// 32-element block (8 elements each, one 16-byte load). grid = rows (any), block 128; K a multiple of 32.
extern "C" __global__ void __launch_bounds__(128)
    kern_quant_mxfp8_rows(const __nv_bfloat16* x, uint8_t* q, uint8_t* sf_rows, int M, int K, int ldx) {
  pdl_wait();
  for (int row = blockIdx.x; row < M; row += gridDim.x) {
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)row * ldx);
    for (int v = threadIdx.x; v < K / 8; v += 128) {
      const uint4 p = src[v];
      float f[8];
      float2 t;
      t = unpack_bf16x2(p.x); f[0] = t.x; f[1] = t.y;
      t = unpack_bf16x2(p.y); f[2] = t.x; f[3] = t.y;
      t = unpack_bf16x2(p.z); f[4] = t.x; f[5] = t.y;
      t = unpack_bf16x2(p.w); f[6] = t.x; f[7] = t.y;
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      int e = 0;
      if (amax > 0.f) {
        int ex;
        const float mant = frexpf(amax, &ex);
        e = mant <= 0.875f ? ex - 9 : ex - 8;
        e = max(-127, min(127, e));
      }
      const float inv = exp2f((float)-e);
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        lo |= (uint32_t)__nv_cvt_float_to_fp8(f[j] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * j);
        hi |= (uint32_t)__nv_cvt_float_to_fp8(f[4 + j] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * j);
      }
      *reinterpret_cast<uint2*>(q + (size_t)row * K + v * 8) = make_uint2(lo, hi);
      if ((v & 3) == 0) sf_rows[(size_t)row * (K / 32) + v / 4] = (uint8_t)(e + 127);
    }
  }
}

// The routed layer's dispatch on one GPU, fused with the activation quantiser: row perm[i] of the expert-sorted MXFP8
// activations = quantised x[i / k], scales in the atom layout over the sorted rows. Four threads share a 32-element
// block (8 elements each, one 16-byte load). grid = entries (tokens * k), block 128; hidden a multiple of 32.
extern "C" __global__ void __launch_bounds__(128)
    kern_moe_gather_quant_mxfp8(const __nv_bfloat16* x, const int* perm, uint8_t* q_perm, uint8_t* sf_perm, int entries,
                                int k, int hidden) {
  pdl_wait();
  const int i = blockIdx.x;
  if (i >= entries) return;
  const int r = perm[i];
  if (r < 0) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(i / k) * hidden);
  const int katoms = (hidden + MX_BK - 1) / MX_BK;
  uint8_t* sf_row = sf_perm + (size_t)(r / 128) * katoms * MX_SF_ATOM + (r % 32) * 16 + ((r / 32) % 4) * 4;
  for (int v = threadIdx.x; v < hidden / 8; v += 128) {
    const uint4 p = src[v];
    float f[8];
    float2 t;
    t = unpack_bf16x2(p.x); f[0] = t.x; f[1] = t.y;
    t = unpack_bf16x2(p.y); f[2] = t.x; f[3] = t.y;
    t = unpack_bf16x2(p.z); f[4] = t.x; f[5] = t.y;
    t = unpack_bf16x2(p.w); f[6] = t.x; f[7] = t.y;
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    int e = 0;
    if (amax > 0.f) {
      int ex;
      const float mant = frexpf(amax, &ex);
      e = mant <= 0.875f ? ex - 9 : ex - 8;
      e = max(-127, min(127, e));
    }
    const float inv = exp2f((float)-e);
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      lo |= (uint32_t)__nv_cvt_float_to_fp8(f[j] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * j);
      hi |= (uint32_t)__nv_cvt_float_to_fp8(f[4 + j] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * j);
    }
    *reinterpret_cast<uint2*>(q_perm + (size_t)r * hidden + v * 8) = make_uint2(lo, hi);
    const int kb = v / 4;
    if ((v & 3) == 0) sf_row[(size_t)(kb / 4) * MX_SF_ATOM + kb % 4] = (uint8_t)(e + 127);
  }
}
