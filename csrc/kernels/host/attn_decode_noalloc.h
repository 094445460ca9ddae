/* Split-KV paged decode attention for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference: it is an addition of this library.
 *
 * Who needs it. The ordinary path (kern_b200.ops.attention.paged_attention, or a manifest's
 * `attn_decode` op) takes its split-KV workspace from the caller: PyTorch's caching allocator or the
 * runtime's scratch buffers. Some hosts cannot provide one at the moment they need attention: a
 * plugin called from inside another engine's stream callback or capture-safe section where
 * cudaMalloc is forbidden, a process whose memory was handed entirely to a pool it does not own, or
 * a C caller that links neither PyTorch nor this library's runtime. For them the workspace lives
 * inside the library, in a fixed device array that every GPU loading the library keeps until exit
 * (about 8.3 MB per GPU), and the call allocates nothing, frees nothing and calls no allocating
 * library routine.
 *
 * Limits. rows = seqs * rows_per_seq. The partial results need rows * hq * splits * head_dim floats;
 * that product may not exceed KERN_NOALLOC_MAX_PARTIAL_FLOATS (2 Mi floats), and
 * rows * hq * splits may not exceed KERN_NOALLOC_MAX_STAT_ROWS (32 Ki). A larger ask is refused with
 * KERN_NOALLOC_TOO_LARGE and nothing is launched. head_dim is 64, 128 or 256.
 *
 * Sharing. Every call on a device uses the same array. Two calls whose kernels may overlap on the GPU
 * (different streams without an ordering between them) race on it; order them on one stream or with
 * an event. The array keeps the previous call's contents; the part that must start at zero (the
 * per-split softmax statistics) is cleared by each call on its stream.
 *
 * First call. The first call on each device looks up the device address of the array and raises the
 * kernels' shared-memory limit, with that device current. Make that first call outside any stream
 * capture; later calls only enqueue a clear, two kernels and nothing else. First calls made from
 * several host threads at once are serialised by a lock inside the library; the calls themselves
 * are not, so the sharing rule above still applies to them.
 */
#ifndef KERN_ATTN_DECODE_NOALLOC_H
#define KERN_ATTN_DECODE_NOALLOC_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KERN_NOALLOC_MAX_PARTIAL_FLOATS (2u * 1024u * 1024u)
#define KERN_NOALLOC_MAX_STAT_ROWS (32u * 1024u)

enum {
  KERN_NOALLOC_OK = 0,
  KERN_NOALLOC_BAD_ARGUMENT = 1, /* a shape the kernels are not built for */
  KERN_NOALLOC_TOO_LARGE = 2,    /* the partials do not fit the built-in workspace */
  KERN_NOALLOC_CUDA_ERROR = 3    /* a CUDA call failed; see kern_noalloc_last_error() */
};

/* q:           bf16, row t holds the hq query heads of token t (row stride q_stride elements)
 * kv_pool:     bf16 [pool_pages][2][hk][page_size][head_dim] (k then v), 16-byte aligned
 * block_table: int32 [seqs][max_pages] page ids; seq_lens: int32 [seqs], context length incl. this step's rows
 * out:         bf16 [rows][out_stride], head h at h*head_dim
 * splits:      2..32 partitions of each sequence's KV range
 * err:         optional device int32: set non-zero if a bounded wait ran out or a page id was out of range
 * stream:      the cudaStream_t to enqueue on (0 = the default stream)
 * Returns one of the codes above; the text of the last failure on this thread is kept. */
int kern_attn_decode_split_noalloc(const void* q, const void* kv_pool, const int32_t* block_table,
                                   const int32_t* seq_lens, void* out, int seqs, int rows_per_seq, int hq, int hk,
                                   int head_dim, int page_size, int max_pages, int pool_pages, int q_stride,
                                   int out_stride, int splits, float softmax_scale, int32_t* err, void* stream);

const char* kern_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
#endif
