// All-gather fused into the tensor-core GEMM (sequence-parallel prefill inside a tensor-parallel group):
//   C[T, N] = G[T, K] . W[N, K]^T, where rank r produced rows [r T/n, (r+1) T/n) of G and the rest is pulled from the
// peers' buffers by the same kernel while the tiles of the local rows are already running. See AgArgs in
// gemm_bf16.cu for the protocol. A cross-rank barrier (kern_peer_barrier) must precede the launch — every rank's slice
// is complete before anyone pulls it — and G alternates between two buffers from call to call, so a rank that runs
// ahead never overwrites rows a peer is still pulling. grid = the SM count in every launch, block 320 (six GEMM warps
// and four gather warps).
// The `_sp` entries are the sequence-parallel form used inside the tensor-parallel decoder: rows owned in 32-row
// sub-blocks dealt round-robin (what kern_sp_reduce_norm leaves behind), readiness by the peers' epoch words instead
// of a barrier kernel, any row count; with the plain store or the SwiGLU epilogue.
// Reference: docs/multi-gpu.md:495-528 (all-gather + GEMM per layer as two steps: nccl_allgather_bf16, then the GEMM).
#define KERN_GEMM_NO_ENTRIES
#include "gemm_bf16.cu"

#define KERN_AG_GEMM_ENTRY(name, BN)                                                                                 \
  extern "C" __global__ void __launch_bounds__(320, 1)                                                               \
      name(const __grid_constant__ CUtensorMap tma_g, const __grid_constant__ CUtensorMap tma_b, void* C, int M,      \
           int N, int K, int ldc, int* err, const unsigned long long* peers, uint32_t* flags, uint32_t* epochs,       \
           int rank, int nranks, int max_blocks) {                                                                   \
    kern::AgArgs ag;                                                                                                 \
    ag.peers = peers; ag.flags = flags; ag.epochs = epochs; ag.rank = rank; ag.nranks = nranks;                      \
    ag.max_blocks = max_blocks;                                                                                      \
    if (M % (nranks * kern::BM) != 0 || (M + kern::BM - 1) / kern::BM > max_blocks) {                                \
      /* a rank's slice must be whole 128-row blocks, and every block needs its counter */                          \
      if (threadIdx.x == 0 && blockIdx.x == 0) kern::set_error(err, kern::ERR_BOUNDS);                               \
      return;                                                                                                        \
    }                                                                                                                \
    kern::gemm_body<BN, 0, false, false, false, true>(&tma_g, &tma_b, C, nullptr, M, N, K, ldc, err, nullptr,        \
                                                      nullptr, kern::ScatterArgs(), nullptr, nullptr, ag);           \
  }

KERN_AG_GEMM_ENTRY(kern_ag_gemm_bf16_tn_n256, 256)
KERN_AG_GEMM_ENTRY(kern_ag_gemm_bf16_tn_n128, 128)

#define KERN_AG_GEMM_SP_ENTRY(name, BN, EPI)                                                                        \
  extern "C" __global__ void __launch_bounds__(320, 1)                                                               \
      name(const __grid_constant__ CUtensorMap tma_g, const __grid_constant__ CUtensorMap tma_b, void* C, int M,      \
           int N, int K, int ldc, int* err, const unsigned long long* peers, uint32_t* flags, uint32_t* epochs,       \
           const uint32_t* ready, const uint32_t* epoch_word, int rank, int nranks, int max_blocks,                   \
           long long timeout_ns, int pushed) {                                                                       \
    kern::AgArgs ag;                                                                                                 \
    ag.peers = peers; ag.flags = flags; ag.epochs = epochs; ag.rank = rank; ag.nranks = nranks;                      \
    ag.max_blocks = max_blocks; ag.ready = ready; ag.epoch_word = epoch_word; ag.timeout_ns = timeout_ns;            \
    ag.pushed = pushed;                                                                                              \
    if ((M + kern::BM - 1) / kern::BM > max_blocks) { /* every block needs its counter */                            \
      if (threadIdx.x == 0 && blockIdx.x == 0) kern::set_error(err, kern::ERR_BOUNDS);                               \
      return;                                                                                                        \
    }                                                                                                                \
    kern::gemm_body<BN, EPI, false, false, false, true>(&tma_g, &tma_b, C, nullptr, M, N, K, ldc, err, nullptr,      \
                                                        nullptr, kern::ScatterArgs(), nullptr, nullptr, ag);         \
  }

KERN_AG_GEMM_SP_ENTRY(kern_ag_gemm_sp_bf16_tn_n256, 256, 0)
KERN_AG_GEMM_SP_ENTRY(kern_ag_gemm_sp_bf16_tn_n128, 128, 0)
KERN_AG_GEMM_SP_ENTRY(kern_ag_gemm_sp_bf16_tn_n64, 64, 0)
KERN_AG_GEMM_SP_ENTRY(kern_ag_gemm_sp_bf16_tn_swiglu_n256, 256, 3)
KERN_AG_GEMM_SP_ENTRY(kern_ag_gemm_sp_bf16_tn_swiglu_n128, 128, 3)
KERN_AG_GEMM_SP_ENTRY(kern_ag_gemm_sp_bf16_tn_swiglu_n64, 64, 3)
