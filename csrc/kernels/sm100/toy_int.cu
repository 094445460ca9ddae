// An exact integer "model" for serving tests: the next token of a sequence is a pure function of what its KV slots
// and its state line hold, so any page handed to the wrong sequence, any slot written at the wrong position, any
// state copied late shows up as a wrong token, not as a small numeric drift. Byte tokens 0..255, end-of-sequence 256.
//
//   slot of token t at position p : WORDS u64 marks, word w = mark(t, p, w)
//   state line of a sequence      : LINE u64, word i = carry ^ (i * K_LINE); carry' = rotl(carry, 11) ^ mark(t, p, 0xffff)
//   S = sum over positions p < L, words w of rotl(slot[p][w], (p + w) & 63)  (+ carry when the model has a line)
//   next = 256 if (S >> 57) % EOS_EVERY == 0 else S & 255
//
// The Python twin (kern_b200/models/toy_int.py) computes the same numbers; the reference has the same idea with its
// own arithmetic (tools/kernels-src/toy.cu, tools/toy/model.py).
#include "common.cuh"

using namespace kern;

namespace {
constexpr int WORDS = 32;
constexpr int LINE = 8;
constexpr unsigned long long K_LINE = 0xD6E8FEB86659FD93ull;
constexpr int EOS_EVERY = 80;

__device__ __forceinline__ unsigned long long fmix(unsigned long long x) {
  x ^= x >> 33; x *= 0xFF51AFD7ED558CCDull;
  x ^= x >> 33; x *= 0xC4CEB9FE1A85EC53ull;
  x ^= x >> 33;
  return x;
}
__device__ __forceinline__ unsigned long long mark(long long t, long long p, int w) {
  return fmix((unsigned long long)t * 0x9FB21C651E98DF25ull ^ (unsigned long long)p * 0xA24BAED4963EE407ull ^
              (unsigned long long)(w + 1) * 0x8CB92BA72F3D8DD7ull);
}
__device__ __forceinline__ unsigned long long rotl(unsigned long long x, int k) {
  k &= 63;
  return k ? (x << k) | (x >> (64 - k)) : x;
}
}  // namespace

// grid rows, block WORDS. kv: [slot][WORDS] u64; slot < 0 skips the row.
extern "C" __global__ void toy_append(const long long* tokens, const long long* positions, const long long* slots,
                                      unsigned long long* kv, int rows, long long kv_slots, int* err) {
  const int r = blockIdx.x;
  if (r >= rows) return;
  const long long s = slots[r];
  if (s < 0) return;
  if (s >= kv_slots) { set_error(err, ERR_BOUNDS); return; }
  kv[(size_t)s * WORDS + threadIdx.x] = mark(tokens[r], positions[r], threadIdx.x);
}

// grid seqs, block 32. Folds this call's rows of every sequence into its line, in order.
extern "C" __global__ void toy_fold(const long long* tokens, const long long* positions, const int* cu_q, const int* lines,
                                    unsigned long long* state, int seqs, int rows_per_seq) {
  const int s = blockIdx.x;
  if (s >= seqs || threadIdx.x != 0) return;
  const int line = lines[s];
  if (line <= 0) return;
  const int r0 = cu_q ? cu_q[s] : s * rows_per_seq, r1 = cu_q ? cu_q[s + 1] : (s + 1) * rows_per_seq;
  unsigned long long* L = state + (size_t)line * LINE;
  unsigned long long c = L[0];
  for (int r = r0; r < r1; ++r) c = rotl(c, 11) ^ mark(tokens[r], positions[r], 0xffff);
  for (int i = 0; i < LINE; ++i) L[i] = c ^ ((unsigned long long)i * K_LINE);
}

// grid seqs, block 256. seq_lens counts this call's rows.
extern "C" __global__ void __launch_bounds__(256)
    toy_predict(const unsigned long long* kv, const int* block_table, const int* seq_lens, const int* lines,
                const unsigned long long* state, const int* cu_q, long long* next, int seqs, int max_pages,
                int page_size) {
  __shared__ unsigned long long red[8];
  const int s = blockIdx.x;
  if (s >= seqs) return;
  // a ragged call names its rows per sequence: a sequence without rows in this call emits nothing (0)
  const int L = (cu_q != nullptr && cu_q[s + 1] == cu_q[s]) ? 0 : seq_lens[s];
  unsigned long long acc = 0;
  for (int i = threadIdx.x; i < L * WORDS; i += 256) {
    const int p = i / WORDS, w = i % WORDS;
    const long long slot = (long long)block_table[(size_t)s * max_pages + p / page_size] * page_size + p % page_size;
    acc += rotl(kv[(size_t)slot * WORDS + w], (p + w) & 63);
  }
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long S = 0;
    for (int i = 0; i < 8; ++i) S += red[i];
    if (lines != nullptr) {
      const int line = lines[s];
      const unsigned long long* Ln = state + (size_t)line * LINE;
      unsigned long long c = Ln[0];
      for (int i = 1; i < LINE; ++i)
        if ((Ln[i] ^ ((unsigned long long)i * K_LINE)) != c) c = ~c;   // a torn line poisons the answer
      if (line > 0) S += c;
    }
    next[s] = L <= 0 ? 0 : (((S >> 57) % EOS_EVERY == 0) ? 256 : (long long)(S & 255));
  }
}
