// Device-side glue of a speculative round (draft -> verify -> accept in one program, one CUDA graph, one host
// sync): the host stages only each sequence's anchor token; the round builds its own rows and reports how many
// tokens it took through the manifest's `count` output. Rollback is free: a paged KV slot is its position, so
// rejected rows are overwritten by the next round.
//
//   kern_spec_splice   ids[i, 0] = anchor[i]; ids[i, 1 + j] = drafts ? drafts[i, j] : mask      (block rows per sequence)
//   kern_spec_rows     positions / KV slots / context lengths of the block rows of every sequence, from the
//                      anchor's position and the page table (the host staged them for one row only)
//   kern_spec_step     the same for draft-chain step j (one row per sequence at position base + j)
//   kern_spec_accept   a = longest prefix of drafts[i] that verify[i] reproduces (row j predicts what follows draft j);
//                      count[i] = a + 1; emitted[i, 0..a] = verify[i, 0..a]; optional wide line table: the sequence's
//                      state line moves to entry a of its cell, every other entry becomes the null line
//   kern_spec_chain    drafts[i, j] = next[i] (collects one chain step's argmax into column j)
// Reference counterparts: tools/kernels-src/spec_round.cu:31-72, tools/kernels-src/markov_rows.cu:42-76.
#include "common.cuh"

using namespace kern;

// grid seqs, block >= block_rows - 1
extern "C" __global__ void kern_spec_splice(const long long* anchor, const long long* drafts, long long* ids, int seqs,
                                            int block_rows, int dstride, long long mask) {
  pdl_wait();
  const int i = blockIdx.x, t = threadIdx.x;
  if (i >= seqs) return;
  if (t == 0) ids[(size_t)i * block_rows] = anchor[i];
  if (t < block_rows - 1) ids[(size_t)i * block_rows + 1 + t] = drafts ? drafts[(size_t)i * dstride + t] : mask;
}

// base_pos[i] = position of the anchor of sequence i. Rows of sequence i sit at i * block_rows + j.
// seq_lens_out[i] = base_pos[i] + block_rows (the context the last row attends to). A position past the sequence's
// page-table row gets slot -1 (nothing appended) and sets the error word.
extern "C" __global__ void kern_spec_rows(const long long* base_pos, const int* block_table, long long* positions,
                                          long long* slots, int* seq_lens_out, int seqs, int block_rows, int max_pages,
                                          int page_size, int* err) {
  pdl_wait();
  const int i = blockIdx.x, j = threadIdx.x;
  if (i >= seqs || j >= block_rows) return;
  const long long p = base_pos[i] + j;
  const long long page_i = p / page_size;
  long long slot = -1;
  if (base_pos[i] < 0) {
    slot = -1;                      // a padding sequence
  } else if (page_i < max_pages) {
    slot = (long long)block_table[(size_t)i * max_pages + page_i] * page_size + p % page_size;
  } else {
    set_error(err, ERR_BOUNDS);
  }
  positions[(size_t)i * block_rows + j] = base_pos[i] < 0 ? 0 : p;
  slots[(size_t)i * block_rows + j] = slot;
  if (j == 0) seq_lens_out[i] = base_pos[i] < 0 ? 0 : (int)(base_pos[i] + block_rows);
}

// One row per sequence at position base_pos[i] + step (a draft chain's step).
extern "C" __global__ void kern_spec_step(const long long* base_pos, const int* block_table, long long* positions,
                                          long long* slots, int* seq_lens_out, int seqs, int step, int max_pages,
                                          int page_size, int* err) {
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= seqs) return;
  const long long b = base_pos[i];
  const long long p = b + step;
  long long slot = -1;
  if (b >= 0) {
    if (p / page_size < max_pages) slot = (long long)block_table[(size_t)i * max_pages + p / page_size] * page_size + p % page_size;
    else set_error(err, ERR_BOUNDS);
  }
  positions[i] = b < 0 ? 0 : p;
  slots[i] = slot;
  seq_lens_out[i] = b < 0 ? 0 : (int)(p + 1);
}

extern "C" __global__ void kern_spec_chain(const long long* next, long long* drafts, int seqs, int column, int dstride) {
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < seqs) drafts[(size_t)i * dstride + column] = next[i];
}

// grid seqs, block 32. line tables are [rows][seqs_max][block_rows] i32 (entry 0 of a cell is the staged line).
extern "C" __global__ void kern_spec_accept(const long long* drafts, const long long* verify, int* count, long long* emitted,
                                            const int* line_in, int* line_adv, int seqs, int block_rows, int dstride,
                                            int line_rows, int seqs_max) {
  pdl_wait();
  const int i = blockIdx.x, t = threadIdx.x;
  if (i >= seqs) return;
  const long long* d = drafts + (size_t)i * dstride;
  const long long* v = verify + (size_t)i * block_rows;
  // lane j < block_rows - 1 votes "draft j was reproduced"; the accepted prefix ends at the first miss
  const bool hit = t < block_rows - 1 ? d[t] == v[t] : false;
  const unsigned miss = ~__ballot_sync(0xffffffffu, hit);
  const int a = min(__ffs(miss) - 1, block_rows - 1);
  if (t == 0) count[i] = a + 1;
  if (emitted != nullptr && t < block_rows) emitted[(size_t)i * block_rows + t] = t <= a ? v[t] : 0;
  if (line_adv != nullptr) {
    for (int r = t; r < line_rows; r += 32) {
      const size_t cell = ((size_t)r * seqs_max + i) * block_rows;
      const int line = line_in[cell];
      for (int e = 0; e < block_rows; ++e) line_adv[cell + e] = e == a ? line : 0;
    }
  }
}

// dst[i] = src[i * stride + column]: one row of every sequence's block (a draft-chain step's token, position, slot).
extern "C" __global__ void kern_spec_column_i64(const long long* src, long long* dst, int seqs, int stride, int column) {
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < seqs) dst[i] = src[(size_t)i * stride + column];
}

// out[i] = max(0, lens[i] - delta) for live sequences (lens[i] > 0), else 0: the context a chain step attends to.
extern "C" __global__ void kern_spec_lens(const int* lens, int* out, int seqs, int delta) {
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < seqs) out[i] = lens[i] > 0 ? max(0, lens[i] - delta) : 0;
}
