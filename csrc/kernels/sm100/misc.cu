// Small data-movement and load-time kernels: row copies, last row of each sequence, own-rows slice
// of a group batch, per-sequence state-line gather/scatter, fills, iota, casts, "+1" weights.
// Reference counterparts: tools/kernels-src/copy_rows.cu:21,30,37; line_copy.cu:17,28;
// weight_prep.cu:24,29,47-67. All take explicit extents and move 16 bytes per thread where the
// row size allows.
#include "common.cuh"

using namespace kern;

// dst[i, :] = src[idx ? idx[i] : i, :]   (row_bytes multiple of 16); idx < 0 skips the row
extern "C" __global__ void kern_copy_rows(const uint8_t* src, uint8_t* dst, const int* idx, int rows,
                                          int row_bytes, int src_stride, int dst_stride) {
  pdl_wait();
  const int r = blockIdx.x;
  if (r >= rows) return;
  const int s = idx ? idx[r] : r;
  if (s < 0) return;
  const uint4* a = reinterpret_cast<const uint4*>(src + (size_t)s * src_stride);
  uint4* b = reinterpret_cast<uint4*>(dst + (size_t)r * dst_stride);
  for (int i = threadIdx.x; i < row_bytes / 16; i += blockDim.x) b[i] = a[i];
}

// dst[s, :] = src[cu_seqlens[s + 1] - 1, :]  — the last row of every sequence of a ragged batch
extern "C" __global__ void kern_last_row(const uint8_t* src, uint8_t* dst, const int* cu_seqlens,
                                         int seqs, int row_bytes) {
  pdl_wait();
  const int s = blockIdx.x;
  if (s >= seqs) return;
  const int r = cu_seqlens[s + 1] - 1;
  if (r < 0) return;
  const uint4* a = reinterpret_cast<const uint4*>(src + (size_t)r * row_bytes);
  uint4* b = reinterpret_cast<uint4*>(dst + (size_t)s * row_bytes);
  for (int i = threadIdx.x; i < row_bytes / 16; i += blockDim.x) b[i] = a[i];
}

// own-rows slice: dst[j, :] = src[blocks[rank] + j, :] for j < blocks[rank+1] - blocks[rank]
extern "C" __global__ void kern_own_rows(const uint8_t* src, uint8_t* dst, const int* blocks, int rank,
                                         int row_bytes) {
  pdl_wait();
  const int lo = blocks[rank], n = blocks[rank + 1] - lo;
  const int j = blockIdx.x;
  if (j >= n) return;
  const uint4* a = reinterpret_cast<const uint4*>(src + (size_t)(lo + j) * row_bytes);
  uint4* b = reinterpret_cast<uint4*>(dst + (size_t)j * row_bytes);
  for (int i = threadIdx.x; i < row_bytes / 16; i += blockDim.x) b[i] = a[i];
}

// per-sequence state lines: gather pool[line[s]] -> span[s], scatter span[s] -> pool[line[s]];
// line 0 is the null line and is skipped
extern "C" __global__ void kern_line_gather(const uint8_t* pool, uint8_t* span, const int* lines,
                                            int seqs, long long line_bytes) {
  pdl_wait();
  const int s = blockIdx.x;
  if (s >= seqs) return;
  const int l = lines[s];
  if (l <= 0) return;
  const uint4* a = reinterpret_cast<const uint4*>(pool + (size_t)l * line_bytes);
  uint4* b = reinterpret_cast<uint4*>(span + (size_t)s * line_bytes);
  for (long long i = blockIdx.y * (long long)blockDim.x + threadIdx.x; i < line_bytes / 16;
       i += (long long)gridDim.y * blockDim.x)
    b[i] = a[i];
}
extern "C" __global__ void kern_line_scatter(uint8_t* pool, const uint8_t* span, const int* lines,
                                             int seqs, long long line_bytes) {
  pdl_wait();
  const int s = blockIdx.x;
  if (s >= seqs) return;
  const int l = lines[s];
  if (l <= 0) return;
  const uint4* a = reinterpret_cast<const uint4*>(span + (size_t)s * line_bytes);
  uint4* b = reinterpret_cast<uint4*>(pool + (size_t)l * line_bytes);
  for (long long i = blockIdx.y * (long long)blockDim.x + threadIdx.x; i < line_bytes / 16;
       i += (long long)gridDim.y * blockDim.x)
    b[i] = a[i];
}

// Batched copies of the pool's copy plans (half pages, state slots): one CTA column per copy.
// plan[c] = {src offset, dst offset, bytes} in bytes relative to `base`, all multiples of 16.
extern "C" __global__ void kern_copy_plan(uint8_t* base, const long long* plan, int copies) {
  const int c = blockIdx.x;
  if (c >= copies) return;
  const long long so = plan[c * 3], d_o = plan[c * 3 + 1], n = plan[c * 3 + 2];
  const uint4* a = reinterpret_cast<const uint4*>(base + so);
  uint4* b = reinterpret_cast<uint4*>(base + d_o);
  for (long long i = blockIdx.y * (long long)blockDim.x + threadIdx.x; i < n / 16;
       i += (long long)gridDim.y * blockDim.x)
    b[i] = a[i];
}

#define KERN_FILL(name, T)                                                                  \
  extern "C" __global__ void name(T* p, long long n, T v) {                                 \
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;             \
         i += (long long)gridDim.x * blockDim.x)                                            \
      p[i] = v;                                                                             \
  }
KERN_FILL(kern_fill_f32, float)
KERN_FILL(kern_fill_i32, int)
KERN_FILL(kern_fill_i64, long long)
KERN_FILL(kern_fill_u8, unsigned char)

extern "C" __global__ void kern_iota_i32(int* p, long long n, int start) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    p[i] = start + (int)i;
}
extern "C" __global__ void kern_cast_bf16_f32(const __nv_bfloat16* src, float* dst, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    dst[i] = __bfloat162float(src[i]);
}
extern "C" __global__ void kern_cast_f32_bf16(const float* src, __nv_bfloat16* dst, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    dst[i] = __float2bfloat16(src[i]);
}
// Gemma-style "+1" weights as f32
extern "C" __global__ void kern_weight_p1_bf16_f32(const __nv_bfloat16* src, float* dst, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    dst[i] = __bfloat162float(src[i]) + 1.f;
}
