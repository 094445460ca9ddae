// Split-KV paged decode attention whose workspace is a fixed device array inside this library, for
// callers that cannot allocate device memory (see attn_decode_noalloc.h for who they are and why).
// No counterpart in the reference. The kernels are the same ones the manifest path launches
// (attn_paged.cu is compiled into this library); only the workspace differs.
#include "attn_decode_noalloc.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <mutex>

#include "../sm100/attn_paged.cu"

namespace {

// partial outputs [rows*hq*splits][head_dim] followed by the per-split (max, sum) pairs
constexpr size_t kPartialFloats = KERN_NOALLOC_MAX_PARTIAL_FLOATS;
constexpr size_t kStatFloats = 2 * (size_t)KERN_NOALLOC_MAX_STAT_ROWS;
static __device__ __align__(256) float g_noalloc_scratch[kPartialFloats + kStatFloats];

constexpr int kMaxDevices = 64;
struct DeviceSetup {
  bool ready = false;
  float* scratch = nullptr;   // device address of g_noalloc_scratch on that device
};
DeviceSetup g_setup[kMaxDevices];
std::mutex g_setup_mutex;   // first calls from several host threads take turns
thread_local char g_last_error[256] = "";

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

int fail(int code, const char* fmt, const char* detail = "") {
  snprintf(g_last_error, sizeof g_last_error, fmt, detail);
  return code;
}

template <typename K>
cudaError_t raise_smem(K kernel, int bytes) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

int smem_for(int d) { return 1024 + (d >= 256 ? 3 : 4) * (2 * 64 * d * 2) + 64 * (d + 8) * 2 + 256; }

// Once per device, with that device current: the host-side name of the array is only a stand-in, the
// kernels need its device address.
int setup_device(int dev) {
  if (dev < 0 || dev >= kMaxDevices) return fail(KERN_NOALLOC_BAD_ARGUMENT, "device index is outside 0..63%s");
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_setup[dev].ready) return KERN_NOALLOC_OK;
  void* p = nullptr;
  cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
  if (e != cudaSuccess) return fail(KERN_NOALLOC_CUDA_ERROR, "cudaGetSymbolAddress: %s", cudaGetErrorString(e));
  if (!g_encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
      return fail(KERN_NOALLOC_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from this driver%s");
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  if ((e = raise_smem(kern_attn_decode_paged_d64, smem_for(64))) != cudaSuccess ||
      (e = raise_smem(kern_attn_decode_paged_d128, smem_for(128))) != cudaSuccess ||
      (e = raise_smem(kern_attn_decode_paged_d256, smem_for(256))) != cudaSuccess)
    return fail(KERN_NOALLOC_CUDA_ERROR, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  g_setup[dev].scratch = static_cast<float*>(p);
  g_setup[dev].ready = true;
  return KERN_NOALLOC_OK;
}

}  // namespace

extern "C" const char* kern_noalloc_last_error(void) { return g_last_error; }

extern "C" int kern_attn_decode_split_noalloc(const void* q, const void* kv_pool, const int32_t* block_table,
                                              const int32_t* seq_lens, void* out, int seqs, int rows_per_seq, int hq,
                                              int hk, int head_dim, int page_size, int max_pages, int pool_pages,
                                              int q_stride, int out_stride, int splits, float softmax_scale,
                                              int32_t* err, void* stream_v) {
  g_last_error[0] = 0;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (!q || !kv_pool || !block_table || !seq_lens || !out) return fail(KERN_NOALLOC_BAD_ARGUMENT, "a required pointer is null%s");
  if (head_dim != 64 && head_dim != 128 && head_dim != 256) return fail(KERN_NOALLOC_BAD_ARGUMENT, "head_dim must be 64, 128 or 256%s");
  if (seqs <= 0 || rows_per_seq <= 0 || hq <= 0 || hk <= 0 || hq % hk || hq / hk > 16)
    return fail(KERN_NOALLOC_BAD_ARGUMENT, "need seqs, rows_per_seq >= 1 and hq a multiple of hk with at most 16 heads per kv head%s");
  if (splits < 2 || splits > 32) return fail(KERN_NOALLOC_BAD_ARGUMENT, "splits must be 2..32%s");
  if (page_size < 8 || !((page_size <= 64 && 64 % page_size == 0) || page_size % 64 == 0))
    return fail(KERN_NOALLOC_BAD_ARGUMENT, "page_size must divide 64 (>= 8) or be a multiple of 64%s");
  if (reinterpret_cast<uintptr_t>(kv_pool) % 16) return fail(KERN_NOALLOC_BAD_ARGUMENT, "kv_pool must be 16-byte aligned%s");
  const size_t rows = (size_t)seqs * rows_per_seq;
  const size_t stat_rows = rows * hq * splits;
  if (stat_rows > KERN_NOALLOC_MAX_STAT_ROWS || stat_rows * head_dim > KERN_NOALLOC_MAX_PARTIAL_FLOATS) {
    snprintf(g_last_error, sizeof g_last_error,
             "rows*hq*splits*head_dim = %zu floats exceeds the built-in workspace of %u floats (or rows*hq*splits = %zu exceeds %u)",
             stat_rows * head_dim, KERN_NOALLOC_MAX_PARTIAL_FLOATS, stat_rows, KERN_NOALLOC_MAX_STAT_ROWS);
    return KERN_NOALLOC_TOO_LARGE;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(KERN_NOALLOC_CUDA_ERROR, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (int rc = setup_device(dev)) return rc;
  float* ws_o = g_setup[dev].scratch;
  float* ws_ml = ws_o + kPartialFloats;

  alignas(64) CUtensorMap map;
  {
    const cuuint64_t dims[2] = {(cuuint64_t)head_dim, (cuuint64_t)pool_pages * 2 * hk * page_size};
    const cuuint64_t strides[1] = {(cuuint64_t)head_dim * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)(page_size < 64 ? page_size : 64)};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(kv_pool), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(KERN_NOALLOC_CUDA_ERROR, "cuTensorMapEncodeTiled rejected the kv pool geometry%s");
  }
  // The statistics of splits that no CTA writes (an empty sequence) must read as "nothing here". A (row, head) is
  // written by every split or by none, so a cleared pair (max 0, sum 0) is never mixed with live ones: the merge
  // sees sum 0 over all splits and writes a zero row, as the allocating path does from its (-inf, 0) pairs.
  e = cudaMemsetAsync(ws_ml, 0, stat_rows * 2 * sizeof(float), stream);
  if (e != cudaSuccess) return fail(KERN_NOALLOC_CUDA_ERROR, "cudaMemsetAsync: %s", cudaGetErrorString(e));

  const int g = hq / hk;
  const int toks_per_blk = 16 / g > 0 ? 16 / g : 1;
  const int nblk = (rows_per_seq + toks_per_blk - 1) / toks_per_blk;
  const dim3 grid(hk * nblk, seqs, splits), block(160);
  const float scale_log2 = softmax_scale * 1.4426950408889634f;
  const __nv_bfloat16* qb = static_cast<const __nv_bfloat16*>(q);
  __nv_bfloat16* ob = static_cast<__nv_bfloat16*>(out);
#define KERN_LAUNCH(D)                                                                                             \
  kern_attn_decode_paged_d##D<<<grid, block, smem_for(D), stream>>>(                                               \
      map, qb, ob, ws_o, ws_ml, block_table, seq_lens, nullptr, nullptr, nullptr, seqs, hq, hk, q_stride,          \
      out_stride, max_pages, page_size, rows_per_seq, splits, pool_pages, scale_log2, err)
  if (head_dim == 64) KERN_LAUNCH(64);
  else if (head_dim == 128) KERN_LAUNCH(128);
  else KERN_LAUNCH(256);
#undef KERN_LAUNCH
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(KERN_NOALLOC_CUDA_ERROR, "attention launch: %s", cudaGetErrorString(e));
  kern_attn_merge_splits<<<(unsigned)(rows * hq), head_dim < 256 ? head_dim : 256, 0, stream>>>(
      ws_o, ws_ml, ob, (int)(rows * hq), hq, head_dim, splits, out_stride);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(KERN_NOALLOC_CUDA_ERROR, "merge launch: %s", cudaGetErrorString(e));
  return KERN_NOALLOC_OK;
}
