// bf16 TN GEMM on the 5th-generation tensor cores: C[M,N] = A[M,K] * W[N,K]^T (+ epilogue).
//
// Serves the manifest extern vocabulary `extern:cublaslt_bf16_tn`, `extern:cublaslt_bf16_tn_acc`
// and `extern:cublas_bf16_tn_f32` (reference: crates/kern-runtime/src/cublas.rs:78-107,242-277,
// 329-378 call cuBLASLt/cuBLAS for these) with one hand-written persistent kernel:
//
//   warp 0      TMA producer: cp.async.bulk.tensor 2-D tiles (128-byte swizzle) into a ring of
//               shared-memory stages, completion on mbarriers
//   warp 1      allocates TMEM, issues tcgen05.mma (128 x BN x 16 per instruction) from one thread,
//               frees each stage / publishes each accumulator with tcgen05.commit
//   warps 2..5  epilogue: tcgen05.ld the f32 accumulator out of TMEM, apply the epilogue, store
//
// Two accumulators live in TMEM (2*BN columns) so the epilogue of tile i overlaps the main loop
// of tile i+1. Grid = min(tiles, SMs): each CTA walks tiles t = blockIdx.x + i*gridDim.x with M
// fastest, so CTAs running at the same time share W tiles through L2.
//
// Epilogues: 0 bf16 store; 1 f32 store; 2 bf16 store of acc + R (R may alias C: the in-place
// residual add, beta = 1); 3 SwiGLU over W = [gate rows ; up rows] (N = 2 x intermediate): each tile
// stages BN/2 gate rows and the matching BN/2 up rows, out[m, n/2] = silu(gate) * up, ldc counts
// output columns. The W descriptor's box is BN/2 rows for this epilogue.
//
// Every mbarrier wait is bounded; a wait that runs out sets *err and the CTA unwinds.
#include "common.cuh"

namespace kern {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row

// MT2: the CTA's tile is 256 rows tall (two 128-row MMAs per K step sharing one B tile). Per FLOP the stage carries a
// third less data from L2 (A 32 KB + B 32 KB per 256x256x64 against 16 + 32 per 128x256x64), which is what bounds the
// 128-row tile at large sizes. The two accumulators fill all 512 TMEM columns, so the epilogue is not overlapped with
// the next tile's MMAs (its loads still are).
template <int BN, bool MT2 = false>
struct GemmCfg {
  static constexpr int kRows = MT2 ? 2 * BM : BM;
  static constexpr int kStageBytesA = kRows * BK * 2;
  static constexpr int kStageBytesB = BN * BK * 2;
  static constexpr int kStageBytes = kStageBytesA + kStageBytesB;
  static constexpr int kStages = MT2 ? 3 : (BN == 256 ? 4 : (BN == 128 ? 6 : 8));
  static constexpr int kAccs = MT2 ? 1 : 2;              // accumulator sets in TMEM
  static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
  // 1024 B of slack for alignment + stages + barriers
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + 256;
};

// EPI 4 (tensor-parallel partial sums): instead of storing C, every row of the tile is pushed over NVLink into the
// staging slot of the rank that will reduce it (the row dealing of the fused all-reduce kernel: row = j + i G,
// owner = (i + j) % nranks, dense index (i / nranks) G + j, parity from that kernel's epoch of column j).
//
// Sequence-parallel form (grid == 0): rows are owned in sub-blocks of kSpRows, sub-block s by rank s % nranks at dense
// index (s / nranks) kSpRows + row % kSpRows; the parity comes from the one epoch word of kern_sp_reduce_norm, which
// reduces the owner's rows only (a reduce-scatter: nothing is sent back). An epilogue warp's 32 rows are one sub-block,
// so they land as 32 consecutive rows of one owner's slot.
constexpr int kSpRows = 32;
struct ScatterArgs {
  const unsigned long long* comm_peers = nullptr;   // every rank's staging buffer, mapped here
  const uint32_t* epochs = nullptr;                 // the reducing kernel's epochs (read only)
  int rank = 0, nranks = 1, grid = 1, slot_rows = 0;
};

// AG (all-gather fused into the GEMM): A is a row-sharded activation, rows [r T/n, (r+1) T/n) produced on rank r. Every
// rank keeps a buffer G of all T rows at the same offsets; its own slice is written by the producing op, and this
// kernel pulls the other slices out of the peers' G (plain 16-byte loads over NVLink, two extra warps per CTA, every
// CTA a share of every 128-row block) while the tensor-core warps already multiply the rows that are here: the tile
// order starts with this rank's own blocks and walks the peers' in the order they are pulled. A block's arrival is a
// counter (every CTA adds one when its share is in place); the TMA producer waits for it — with a limit — before the
// first load of a tile from that block. Counters only grow: launch e of a grid of g CTAs brings each to e g, so
// nothing is reset and captured graphs replay; the grid size must therefore be the same in every launch.
KERN_DEVICE int num_m_of(int M, int nranks) { return (M / nranks + BM - 1) / BM; }

//
// Sequence-parallel form (`ready` set): G's rows are owned in sub-blocks of kSpRows (sub-block s by rank s % nranks, the
// layout kern_sp_reduce_norm leaves), so every 128-row block holds rows of up to four owners and none is local: the
// gather warps first wait (bounded) until every peer's `ready` word has reached this rank's own epoch, i.e. the peer's
// rows of this call are final, then pull each block's foreign rows in block order while the tiles of the blocks
// already here run. No barrier kernel before or after: the reduce kernel of the next call lines the ranks up again
// before anyone rewrites a row.
constexpr int kGatherWarps = 4;
constexpr int kAgWindow = 8;     // 128-row blocks per window of the tile order
struct AgArgs {
  const unsigned long long* peers = nullptr;   // G of every rank, mapped here (this rank's own included)
  uint32_t* flags = nullptr;                   // [max_blocks] arrival counters (local)
  uint32_t* epochs = nullptr;                  // [grid] launches seen by each CTA (local)
  int rank = 0, nranks = 1, max_blocks = 0;
  const uint32_t* ready = nullptr;             // sequence-parallel: [nranks] epochs at which each rank's rows were final
  const uint32_t* epoch_word = nullptr;        //   and this rank's own epoch
  int pushed = 0;                              //   1: the owners pushed their rows here already; only wait for the flags
  long long timeout_ns = 2000000000ll;
};

// EP (expert parallel over sharded tokens; both forms are GROUPED):
//   EP == 1, dispatch fused into the routed GEMM: the A operand is the expert-sorted activation buffer `xg`, and the
//     rows are not there yet when the kernel starts. Row r of xg is token src_tok[r] (a global index: home rank =
//     token / rows_per_rank; -1: padding), and the gather warps of the AG form pull every row straight out of its home
//     rank's exported activation buffer (16-byte peer loads over NVLink, local rows through the same code) while the
//     tensor-core warps already multiply the 128-row blocks that have arrived; the arrival counters and the producer's
//     bounded wait are the AG form's. Needs the aligned plan (every tile starts on a 128-row boundary of xg).
//   EPI == 5, combine fused into the routed GEMM's epilogue: row r of the result goes from TMEM straight into slot
//     (token, choice) of the return buffer on the token's home rank (bf16, whole 128-byte lines over NVLink through the
//     same shared-memory staging as EPI 4; a slot has exactly one writer, local tokens take the same path). When the
//     last CTA of the grid is done it publishes this rank's epoch into every rank's `done` words; the home rank's
//     finalize kernel waits for all of them and then forms the top-k weighted sum of its k slots. (Adding weighted f32
//     rows into an accumulator on the home rank with red.add instead was measured first: 16-byte reductions over
//     NVLink made the routed layer 25-45 % slower than the un-fused chain.)
struct EpArgs {
  const unsigned long long* x_peers = nullptr;    // dispatch: every rank's activation buffer [rows_per_rank, K]
  __nv_bfloat16* xg = nullptr;                    //           this rank's expert-sorted rows (the A operand)
  const int* src_tok = nullptr;                   // both: global token of each expert-sorted row, -1 for padding
  const int* row_choice = nullptr;                // combine: which of its token's k choices each expert-sorted row is
  const unsigned long long* ret_peers = nullptr;  //          every rank's return buffer [rows_per_rank, k, N] bf16
  const unsigned long long* done_peers = nullptr; //          every rank's done words [nranks]
  uint32_t* state = nullptr;                      //          {CTAs finished, epoch} (local)
  int rows_per_rank = 1, rank = 0, nranks = 1, k = 1;
};

// GROUPED: the M tiles come from a device table of int4 {expert, first row, rows (<= BM), -} built by the MoE
// planner (`tile_count` of them); A rows are the expert-sorted activations, B is a 3-D map [K, N, experts].
// A tile's load may run into the next expert's rows; the epilogue stores only the tile's own rows.
// FP8: A and B hold e4m3 bytes (a swizzle row is 128 elements, the instruction is kind::f8f6f4 with K = 32), the
// accumulator is scaled by *scale_a * *scale_b (per-tensor scales) before the epilogue's conversion.
template <int BN, int EPI, bool GROUPED = false, bool FP8 = false, bool MT2 = false, bool AG = false, int EP = 0>
__device__ __forceinline__ void gemm_body(const CUtensorMap* tma_a, const CUtensorMap* tma_b,
                                          void* Cv, const void* Rv,
                                          int M, int N, int K, int ldc, int* err,
                                          const int* tile_table = nullptr, const int* tile_count = nullptr,
                                          ScatterArgs sc = ScatterArgs(), const float* scale_a = nullptr,
                                          const float* scale_b = nullptr, AgArgs ag = AgArgs(), EpArgs ep = EpArgs()) {
  using Cfg = GemmCfg<BN, MT2>;
  constexpr int kStages = Cfg::kStages;
  constexpr int BMT = Cfg::kRows;
  static_assert(!(MT2 && (GROUPED || EPI == 4 || BN != 256)), "the 256-row tile exists for the plain 256-wide GEMM");
  static_assert(!(AG && (FP8 || MT2)) && (!(AG && GROUPED) || EP == 1), "the all-gather form exists for the plain bf16 GEMM");
  static_assert((EP != 1 || (AG && GROUPED)) && (EPI != 5 || GROUPED), "the expert-parallel forms are routed GEMMs");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * Cfg::kStageBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tfull_bar = empty_bar + kStages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_n = (N + BN - 1) / BN;
  constexpr int BKE = FP8 ? 2 * BK : BK;   // elements of one 128-byte swizzle row
  const int num_kb = (K + BKE - 1) / BKE;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4);  // one arrive per epilogue warp
    }
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
  if (threadIdx.x == 0) {
    tma_prefetch_desc(tma_a);
    tma_prefetch_desc(tma_b);
  }
  pdl_wait();  // everything above touched only this CTA's own state and the descriptors
  const int num_m = GROUPED ? *tile_count : (M + BMT - 1) / BMT;
  const int num_tiles = num_m * num_n;
  // tile t -> (first row, row bound, n block, expert)
  // AG: blocks per rank, this rank's first block, and the counter value that says "every CTA's share of the block is in"
  const int ag_bpr = AG ? ((EP == 1 || ag.ready != nullptr) ? 0 : num_m_of(M, ag.nranks)) : 0;
  // the block this rank's tile order and pulls start from: its own rows (contiguous slices), or a rank-dependent
  // offset so that the ranks pull from different owners at any one time (sequence-parallel sub-blocks); the routed
  // form pulls its expert-sorted rows in ascending order, so its tiles start at block 0
  const int ag_first = (AG && EP != 1) ? (ag_bpr ? ag.rank * ag_bpr : (int)(((long long)ag.rank * num_m) / ag.nranks)) : 0;
  const int bpr_div = ag_bpr ? ag_bpr : 1;     // divisor where the blocks-per-rank form of the expression is not taken
  uint32_t ag_want = 0;
  if constexpr (AG) {
    // the routed form counts rows (every launch adds BM to each counter), the others the CTAs that have put their share in
    ag_want = (ag.epochs[blockIdx.x] + 1u) * (EP == 1 ? (uint32_t)BM : gridDim.x);
    __syncthreads();      // every thread has read this CTA's launch count before the gather warps can write the next one
  }
  auto tile_of = [&](int t, int& row0, int& row_end, int& n_blk, int& expert) {
    int mt = t % num_m;
    n_blk = t / num_m;
    if constexpr (AG) {
      // Blocks in the order they arrive (this rank's first block first), kAgWindow of them at a time with the row
      // blocks fastest inside a window: CTAs that run together then share a few W tiles through L2 (with the columns
      // fastest every wave would stream the whole of W), and no tile waits for a block far down the pull order.
      const int per_win = kAgWindow * num_n;
      const int w = t / per_win, r = t - w * per_win;
      const int m0 = w * kAgWindow, wm = min(kAgWindow, num_m - m0);
      mt = (m0 + r % wm + ag_first) % num_m;
      n_blk = r / wm;
    }
    if constexpr (GROUPED) {
      const int4 e = reinterpret_cast<const int4*>(tile_table)[mt];
      expert = e.x; row0 = e.y; row_end = min(M, e.y + e.z);
    } else {
      expert = 0; row0 = mt * BMT; row_end = M;
    }
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int row0, row_end, n_blk, expert;
        tile_of(t, row0, row_end, n_blk, expert);
        if constexpr (AG) {
          const int blk = row0 / BM;
          if (ag_bpr == 0 || blk / bpr_div != ag.rank) {       // a peer's rows: wait until every CTA has put its share of the block here
            bool here = false;
            for (uint32_t i = 0; i < (1u << 22) && !here; ++i) {
              here = ld_acquire_sys(ag.flags + blk) >= ag_want;
              if (!here) { if ((i & 0xff) == 0xff && *abort_flag != 0) break; __nanosleep(100); }
            }
            if (!here) {
              set_error(err, ERR_WAIT_PEER + (ag_bpr ? blk / bpr_div : ag.nranks));
              *abort_flag = 1;
              break;
            }
            asm volatile("fence.proxy.async;" ::: "memory");   // the rows were written by ordinary stores; TMA reads them next
          }
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
            set_error(err, ERR_WAIT_EMPTY);
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* sa = tiles + stage * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kStageBytesA;
          mbar_expect_tx(&full_bar[stage], Cfg::kStageBytes);
          tma_load_2d(sa, tma_a, kb * BKE, row0, &full_bar[stage]);
          auto load_b = [&](uint8_t* dst, int n_row) {
            if constexpr (GROUPED) tma_load_3d(dst, tma_b, kb * BKE, n_row, expert, &full_bar[stage]);
            else tma_load_2d(dst, tma_b, kb * BKE, n_row, &full_bar[stage]);
          };
          if constexpr (EPI == 3) {
            // W = [gate rows ; up rows]: this tile's B rows are BN/2 gate rows then the matching BN/2 up rows
            load_b(sb, n_blk * (BN / 2));
            load_b(sb + (BN / 2) * BK * 2, N / 2 + n_blk * (BN / 2));
          } else {
            load_b(sb, n_blk * BN);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      // e4m3 is format 0 of kind::f8f6f4, bf16 format 1 of kind::f16: the descriptors differ only in those fields
      constexpr uint32_t idesc = FP8 ? ((1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24))
                                     : umma_idesc_bf16(BM, BN);
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
          const uint32_t sa = smem_u32(tiles + stage * Cfg::kStageBytes);
          const uint32_t sb = sa + Cfg::kStageBytesA;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            if constexpr (FP8)
              umma_f8f6f4(d_tmem, umma_desc_sw128(sa + k * 32), umma_desc_sw128(sb + k * 32), idesc, (kb | k) != 0);
            else
              umma_bf16(d_tmem, umma_desc_sw128(sa + k * 32), umma_desc_sw128(sb + k * 32), idesc, (kb | k) != 0);
            if constexpr (MT2)      // rows 128..255 of the tile: the A sub-tile 16 KB further on, the next BN TMEM columns
              umma_bf16(d_tmem + BN, umma_desc_sw128(sa + BM * BK * 2 + k * 32), umma_desc_sw128(sb + k * 32), idesc,
                        (kb | k) != 0);
          }
          tc_commit(&empty_bar[stage]);  // stage is free once these MMAs have read it
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit(&tfull_bar[acc]);
        if (++acc == Cfg::kAccs) { acc = 0; acc_phase ^= 1; }
      }
    }
    __syncwarp();
  } else if (warp >= 6) {
    // ---------------- gather warps 6.. (AG only): pull the peers' rows into this rank's G ----------------
    if constexpr (AG) {
      constexpr int GT = kGatherWarps * 32;
      const int gt = threadIdx.x - 192;                      // 0..GT-1
      if constexpr (EP == 1) {
        // Routed form: a warp per row. Row r of the sorted buffer is token src_tok[r] on its home rank; the warp copies
        // its K * 2 bytes (eight 16-byte loads in flight per lane, the next eight issued before the stores of the last),
        // and then adds one to the row's block counter; padding rows count at once. A block is ready at BM arrivals.
        const int gw = blockIdx.x * kGatherWarps + (warp - 6), GW = gridDim.x * kGatherWarps;
        const int row_vecs = K * 2 / 16, total_rows = num_m * BM;
        for (int b = num_m + gw * 32 + lane; b < ag.max_blocks; b += GW * 32) atomicAdd(ag.flags + b, (uint32_t)BM);   // unused this launch
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
            const uint8_t* src = reinterpret_cast<const uint8_t*>(ep.x_peers[tok / ep.rows_per_rank]) +
                                 (size_t)(tok % ep.rows_per_rank) * row_vecs * 16;
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(ep.xg) + (size_t)r * row_vecs * 16);
            uint4 xa[8], xb[8];
            const bool ok_row = KERN_CHECK(src, (size_t)row_vecs * 16, SITE_EP_PULL) && KERN_CHECK(dst, (size_t)row_vecs * 16, SITE_MOE_GATHER);
            if (ok_row) ld8(src, lane, xa);
            for (int v0 = lane; ok_row && v0 < row_vecs; v0 += 256) {
              if (v0 + 256 < row_vecs) ld8(src, v0 + 256, xb);
#pragma unroll
              for (int q = 0; q < 8; ++q)
                if (v0 + q * 32 < row_vecs) dst[v0 + q * 32] = xa[q];
#pragma unroll
              for (int q = 0; q < 8; ++q) xa[q] = xb[q];
            }
            __threadfence();
            asm volatile("fence.proxy.async;" ::: "memory");
          }
          __syncwarp();
          if (lane == 0) atomicAdd(ag.flags + (r >> 7), 1u);
        }
        asm volatile("bar.sync 1, %0;" ::"n"(GT) : "memory");
        if (gt == 0) ag.epochs[blockIdx.x] = ag_want / BM;
      } else {
      uint8_t* mine = reinterpret_cast<uint8_t*>(ag.peers[ag.rank]);
      const bool sp = ag.ready != nullptr;
      if (sp) {
        // every peer's rows of this call are final once its `ready` word has reached this rank's own epoch
        const uint32_t e = *reinterpret_cast<const volatile uint32_t*>(ag.epoch_word);
        if (gt < ag.nranks && gt != ag.rank) {
          const uint64_t t0 = globaltimer_ns();
          while ((int32_t)(ld_acquire_sys(ag.ready + gt) - e) < 0) {
            if (*abort_flag != 0) break;
            if ((long long)(globaltimer_ns() - t0) > ag.timeout_ns) {
              set_error(err, ERR_WAIT_PEER + gt);
              *abort_flag = 1;
              break;
            }
            __nanosleep(40);
          }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(GT) : "memory");
      }
      // blocks nobody gathers in this launch (own rows, blocks past the last row) arrive at once: every counter moves
      // by the grid size in every launch, whatever the row count
      for (int b = gt; b < ag.max_blocks; b += GT) {
        const bool remote = b < num_m && !ag.pushed && (sp || b / bpr_div != ag.rank);
        if (!remote) atomicAdd(ag.flags + b, 1u);
      }
      // The blocks to pull, in the order the tiles will want them, form one run of 16-byte vectors that is cut into units
      // of eight vectors per thread over the whole grid (a unit usually spans two or three blocks). The loads of unit
      // u + 1 are issued before the stores of unit u, so a thread keeps up to sixteen peer loads in flight: a peer load
      // takes a few microseconds, and the link is only busy while about latency x bandwidth bytes are outstanding.
      // A block's counter moves once every unit that touches the block has been stored.
      const size_t row_vecs = (size_t)K * 2 / 16;
      const size_t vecs = (size_t)BM * row_vecs, stride = (size_t)gridDim.x * GT, span = stride * 8;
      const int pull_blocks = ag.pushed ? 0 : (sp ? num_m : num_m - ag_bpr);
      const size_t total = (size_t)pull_blocks * vecs;
      const int units = (*abort_flag != 0) ? 0 : (int)((total + span - 1) / span);
      auto block_at = [&](int i) { return ((sp ? 0 : ag_bpr) + i + ag_first) % num_m; };   // i-th block in pull order
      // where vector v of block b comes from (null: it is this rank's own, or past the last row)
      auto source = [&](int b, size_t v) -> const uint8_t* {
        if (!sp) return reinterpret_cast<const uint8_t*>(ag.peers[b / bpr_div]) + (size_t)b * BM * K * 2 + v * 16;
        const int row = b * BM + (int)(v / row_vecs);
        const int owner = (row / kSpRows) % ag.nranks;
        if (row >= M || owner == ag.rank) return nullptr;
        return reinterpret_cast<const uint8_t*>(ag.peers[owner]) + (size_t)b * BM * K * 2 + v * 16;
      };
      auto load = [&](int u, uint4 (&x)[8], uint32_t& have) {
        const size_t l0 = (size_t)u * span + (size_t)blockIdx.x * GT + gt;
        have = 0;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const size_t l = l0 + q * stride;
          if (l < total) {
            const int i = (int)(l / vecs);
            const uint8_t* src = source(block_at(i), l - (size_t)i * vecs);
            if (src != nullptr) {
              have |= 1u << q;
              asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                           : "=r"(x[q].x), "=r"(x[q].y), "=r"(x[q].z), "=r"(x[q].w) : "l"(src));
            }
          }
        }
      };
      uint4 xa[8], xb[8];
      uint32_t ha = 0, hb = 0;
      int signalled = 0;                                                   // blocks (in pull order) whose counter has moved
      if (units > 0) load(0, xa, ha);
      for (int u = 0; u < units; ++u) {
        if (u + 1 < units) load(u + 1, xb, hb);
        const size_t l0 = (size_t)u * span + (size_t)blockIdx.x * GT + gt;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          if (ha & (1u << q)) {
            const size_t l = l0 + q * stride;
            const int i = (int)(l / vecs);
            *reinterpret_cast<uint4*>(mine + (size_t)block_at(i) * BM * K * 2 + (l - (size_t)i * vecs) * 16) = xa[q];
          }
        }
        const size_t covered = (size_t)(u + 1) * span;
        const int complete = covered >= total ? pull_blocks : (int)(covered / vecs);
        if (complete > signalled) {                                        // this CTA's share of these blocks is in place
          __threadfence();
          asm volatile("fence.proxy.async;" ::: "memory");
          asm volatile("bar.sync 1, %0;" ::"n"(GT) : "memory");          // all gather warps are done with them
          if (gt == 0)
            for (int i = signalled; i < complete; ++i) atomicAdd(ag.flags + block_at(i), 1u);
          signalled = complete;
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) xa[q] = xb[q];
        ha = hb;
      }
      if (gt == 0) ag.epochs[blockIdx.x] = ag_want / gridDim.x;
      }   // !EP
    }
  } else {
    // ---------------- epilogue warps 2..5 ----------------
    const int quarter = warp & 3;  // TMEM lanes 32*quarter .. +31 are this warp's
    const float out_scale = FP8 ? scale_a[0] * scale_b[0] : 1.f;
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
#pragma unroll 1
      for (int hh = 0; hh < (MT2 ? 2 : 1); ++hh) {     // the 256-row tile drains its two 128-row accumulators in turn
      const int row = row0 + hh * BM + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (MT2 ? hh : acc) * BN;
      if constexpr (EPI == 3) {
        // SwiGLU: accumulator columns [0, BN/2) are gate, [BN/2, BN) the matching up columns
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          uint32_t g[32], u[32];
          tmem_ld_32x32(t_row + c * 32, g);
          tmem_ld_32x32(t_row + BN / 2 + c * 32, u);
          tmem_ld_wait();
          const int col = n_blk * (BN / 2) + c * 32;   // output column
          if (row < row_end && col < N / 2) {
            __nv_bfloat16* C = reinterpret_cast<__nv_bfloat16*>(Cv) + (size_t)row * ldc + col;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (col + v * 8 < N / 2) {
                float f[8];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  f[j] = silu(__uint_as_float(g[v * 8 + j])) * __uint_as_float(u[v * 8 + j]);
                uint4 o;
                o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
                o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
                *reinterpret_cast<uint4*>(C + v * 8) = o;
              }
            }
          }
        }
      } else if constexpr (EPI == 4 || EPI == 5) {
        // Rows go to the rank that reduces them. A lane first works out where its own row lands (once per tile);
        // then, 64 columns at a time, the warp parks its 32 x 64 block in shared memory and writes it out four rows
        // per instruction, eight lanes per row: every peer store covers a whole 128-byte line.
        uint8_t* stage = smem + kStages * Cfg::kStageBytes + 512 + quarter * (32 * 144 + 256);
        unsigned long long* rowptr = reinterpret_cast<unsigned long long*>(stage + 32 * 144);
        {
          unsigned long long dst = 0;
          if constexpr (EPI == 5) {
            // the row's slot (token, choice) in the return buffer of the token's home rank
            if (row < row_end) {
              const int tok = ep.src_tok[row];
              if (tok >= 0)
                dst = ep.ret_peers[tok / ep.rows_per_rank] +
                      2ull * (((size_t)(tok % ep.rows_per_rank) * ep.k + ep.row_choice[row]) * (size_t)N);
              if (dst != 0 && !KERN_CHECK(reinterpret_cast<const void*>(dst), (size_t)N * 2, SITE_EP_SLOT)) dst = 0;
            }
          } else if (row < row_end) {
            int j, owner, idx;
            if (sc.grid == 0) {          // sequence-parallel: sub-blocks of kSpRows rows, one epoch word
              const int sb = row / kSpRows;
              j = 0; owner = sb % sc.nranks; idx = (sb / sc.nranks) * kSpRows + row % kSpRows;
            } else {
              j = row % sc.grid;
              const int i = row / sc.grid;
              owner = (i + j) % sc.nranks; idx = (i / sc.nranks) * sc.grid + j;
            }
            if (idx >= sc.slot_rows) {
              set_error(err, ERR_BOUNDS);
            } else {
              const uint32_t parity = (sc.epochs[j] + 1) & 1;
              const size_t slot_elems = (size_t)sc.slot_rows * N;
              dst = sc.comm_peers[owner] +
                    2ull * (parity * ((size_t)sc.nranks * slot_elems) + sc.rank * slot_elems + (size_t)idx * N);
            }
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
          if constexpr (EPI == 0 || EPI == 2) {
            __nv_bfloat16* C = reinterpret_cast<__nv_bfloat16*>(Cv) + (size_t)row * ldc + col;
            const __nv_bfloat16* R =
                reinterpret_cast<const __nv_bfloat16*>(Rv) + (size_t)row * ldc + col;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (col + v * 8 < N) {
                float f[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[v * 8 + j]) * out_scale;
                if constexpr (EPI == 2) {
                  uint4 old = *reinterpret_cast<const uint4*>(R + v * 8);
                  float2 a = unpack_bf16x2(old.x), b = unpack_bf16x2(old.y),
                         cc = unpack_bf16x2(old.z), d = unpack_bf16x2(old.w);
                  f[0] += a.x; f[1] += a.y; f[2] += b.x; f[3] += b.y;
                  f[4] += cc.x; f[5] += cc.y; f[6] += d.x; f[7] += d.y;
                }
                uint4 o;
                o.x = pack_bf16x2(f[0], f[1]);
                o.y = pack_bf16x2(f[2], f[3]);
                o.z = pack_bf16x2(f[4], f[5]);
                o.w = pack_bf16x2(f[6], f[7]);
                *reinterpret_cast<uint4*>(C + v * 8) = o;
              }
            }
          } else if constexpr (EPI == 1) {
            float* C = reinterpret_cast<float*>(Cv) + (size_t)row * ldc + col;
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              if (col + v * 4 < N) {
                float4 o = make_float4(__uint_as_float(r[v * 4]) * out_scale, __uint_as_float(r[v * 4 + 1]) * out_scale,
                                       __uint_as_float(r[v * 4 + 2]) * out_scale,
                                       __uint_as_float(r[v * 4 + 3]) * out_scale);
                *reinterpret_cast<float4*>(C + v * 4) = o;
              }
            }
          }
        }
      }
      }
      }   // hh
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      if (++acc == Cfg::kAccs) { acc = 0; acc_phase ^= 1; }
    }
  }

  // ---------------- teardown ----------------
  if constexpr (EPI == 4 || EPI == 5) __threadfence_system();   // the pushed rows are on their way before the kernel is done
  pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  if constexpr (EPI == 5) {
    // the last CTA to get here publishes this rank's epoch: every add of this launch is ordered before it
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
    // give loads that were in flight time to land before the CTA (and its shared memory) retires
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

#ifndef KERN_GEMM_NO_ENTRIES
#define KERN_GEMM_ENTRY(name, BN, EPI)                                                        \
  extern "C" __global__ void __launch_bounds__(192, 1)                                        \
      name(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, \
           void* C, const void* R, int M, int N, int K, int ldc, int* err) {                  \
    kern::gemm_body<BN, EPI>(&tma_a, &tma_b, C, R, M, N, K, ldc, err);                        \
  }

#define KERN_GEMM_ENTRY_M256(name, EPI)                                                       \
  extern "C" __global__ void __launch_bounds__(192, 1)                                        \
      name(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, \
           void* C, const void* R, int M, int N, int K, int ldc, int* err) {                  \
    kern::gemm_body<256, EPI, false, false, true>(&tma_a, &tma_b, C, R, M, N, K, ldc, err);   \
  }

KERN_GEMM_ENTRY_M256(kern_gemm_bf16_tn_m256_n256, 0)
KERN_GEMM_ENTRY_M256(kern_gemm_bf16_tn_acc_m256_n256, 2)
KERN_GEMM_ENTRY_M256(kern_gemm_bf16_tn_swiglu_m256_n256, 3)
KERN_GEMM_ENTRY(kern_gemm_bf16_tn_n256, 256, 0)
KERN_GEMM_ENTRY(kern_gemm_bf16_tn_n128, 128, 0)
KERN_GEMM_ENTRY(kern_gemm_bf16_tn_n64, 64, 0)
KERN_GEMM_ENTRY(kern_gemm_bf16_tn_n32, 32, 0)
KERN_GEMM_ENTRY(kern_gemm_bf16_tn_f32_n256, 256, 1)
KERN_GEMM_ENTRY(kern_gemm_bf16_tn_f32_n128, 128, 1)
KERN_GEMM_ENTRY(kern_gemm_bf16_tn_f32_n64, 64, 1)
KERN_GEMM_ENTRY(kern_gemm_bf16_tn_acc_n256, 256, 2)
KERN_GEMM_ENTRY(kern_gemm_bf16_tn_acc_n128, 128, 2)
KERN_GEMM_ENTRY(kern_gemm_bf16_tn_acc_n64, 64, 2)
KERN_GEMM_ENTRY(kern_gemm_bf16_tn_acc_n32, 32, 2)
KERN_GEMM_ENTRY(kern_gemm_bf16_tn_swiglu_n256, 256, 3)
KERN_GEMM_ENTRY(kern_gemm_bf16_tn_swiglu_n128, 128, 3)
KERN_GEMM_ENTRY(kern_gemm_bf16_tn_swiglu_n64, 64, 3)
#endif  // KERN_GEMM_NO_ENTRIES
