// Tensor-parallel GEMM whose epilogue is the first half of the reduce-scatter: each rank's partial tile goes
// straight from TMEM over NVLink into the reducing rank's staging slot (plain peer stores, 16 bytes each), so the
// transfer of tile t overlaps the tensor-core work of tile t+1 and the partial sums never touch local HBM. The
// reduction, residual add, RMSNorm and the all-gather of the new rows are kern_tp_allreduce_residual_norm in mode 2,
// launched next on the same stream.
// The reference does this as a library GEMM followed by an NCCL reduce-scatter (docs/multi-gpu.md:495-528).
#define KERN_GEMM_NO_ENTRIES
#include "gemm_bf16.cu"

#define KERN_TP_GEMM_ENTRY(name, BN)                                                                              \
  extern "C" __global__ void __launch_bounds__(192, 1)                                                            \
      name(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, int M, int N,      \
           int K, int* err, const unsigned long long* comm_peers, const uint32_t* epochs, int rank, int nranks,     \
           int grid, int slot_rows) {                                                                              \
    kern::ScatterArgs sc;                                                                                          \
    sc.comm_peers = comm_peers; sc.epochs = epochs; sc.rank = rank; sc.nranks = nranks; sc.grid = grid;            \
    sc.slot_rows = slot_rows;                                                                                      \
    kern::gemm_body<BN, 4>(&tma_a, &tma_b, nullptr, nullptr, M, N, K, N, err, nullptr, nullptr, sc);               \
  }

KERN_TP_GEMM_ENTRY(kern_tp_gemm_scatter_bf16_n256, 256)
KERN_TP_GEMM_ENTRY(kern_tp_gemm_scatter_bf16_n128, 128)
KERN_TP_GEMM_ENTRY(kern_tp_gemm_scatter_bf16_n64, 64)
