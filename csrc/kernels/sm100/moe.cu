// Mixture-of-experts routing and the routed (grouped) tcgen05 GEMM.
//
//   kern_moe_route_f32      router scores -> top-k expert ids and weights per token (sigmoid or softmax scoring,
//                           optional selection bias, renormalise, scale)
//   kern_moe_plan           counts per expert -> row offsets, the permuted row of every (token, choice), and the
//                           M-tile table the grouped GEMM walks; experts outside [e_lo, e_hi) belong to another rank
//   kern_moe_gather_bf16    x_perm[perm[t, j]] = x[t]
//   kern_moe_gemm_*         C_perm = A_perm . W[expert]^T over the tile table (store / SwiGLU epilogues)
//   kern_moe_combine_bf16   out[t] = (acc ? out[t] : 0) + sum_j w[t, j] * y_perm[perm[t, j]]  (+ shared[t])
//
// Reference counterparts: tools/kernels-src/topk_row.cu:21 (top-k per row); the routed batched GEMMs the reference
// takes as prebuilt blobs (kernel_index/trtllm_bmm_*.toml) are written here on the same tcgen05 body as the dense GEMM.
#define KERN_GEMM_NO_ENTRIES
#include "gemm_bf16.cu"

using namespace kern;

// One warp per token; E <= 1024. mode 0: sigmoid scores, mode 1: softmax over all experts.
// Selection uses score + bias (bias may be null); the weight is the unbiased score. renorm: weights sum to 1.
extern "C" __global__ void __launch_bounds__(128)
    kern_moe_route_f32(const float* logits, const float* bias, int* topk_ids, float* topk_w, int tokens, int experts,
                       int k, int mode, int renorm, float scale, int ld) {
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= tokens) return;
  constexpr int PER = 32;   // up to 1024 experts
  float sc[PER], sel[PER];
  const float* row = logits + (size_t)t * ld;
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = i * 32 + lane;
    sc[i] = e < experts ? row[e] : -INFINITY;
    mx = fmaxf(mx, sc[i]);
  }
  if (mode == 1) {
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = i * 32 + lane;
      sc[i] = e < experts ? __expf(sc[i] - mx) : 0.f;
      sum += sc[i];
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int i = 0; i < PER; ++i) sc[i] /= sum;
  } else {
#pragma unroll
    for (int i = 0; i < PER; ++i) sc[i] = 1.f / (1.f + __expf(-sc[i]));
  }
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = i * 32 + lane;
    sel[i] = e < experts ? sc[i] + (bias ? bias[e] : 0.f) : -INFINITY;
  }
  float wsum = 0.f;
  float my_w = 0.f;
  int my_id = 0;
  for (int j = 0; j < k; ++j) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = i * 32 + lane;
      if (sel[i] > best) { best = sel[i]; bi = e; }   // lowest index wins ties within a lane (ascending scan)
    }
    // warp arg-max, ties -> lowest expert id
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    float w = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i)
      if (i * 32 + lane == bi) { w = sc[i]; sel[i] = -INFINITY; }
    w = warp_sum(w);
    wsum += w;
    if (lane == j) { my_w = w; my_id = bi; }
  }
  if (lane < k) {
    const float w = renorm ? my_w / (wsum + 1e-20f) : my_w;
    topk_ids[(size_t)t * k + lane] = my_id;
    topk_w[(size_t)t * k + lane] = w * scale;
  }
}

// Single CTA (block 1024). entries = tokens * k. Outputs:
//   perm[entries]      permuted row of each (token, choice), -1 when the expert is not local
//   offsets[E_local+1] first permuted row of every local expert
//   tiles[int4]        {local expert, first row, rows, 0} per M tile of `bm` rows; tile_count[0] = how many
//   rows_out[0]        total permuted rows
//
// `align`: every expert's first row is rounded up to a multiple of it (the block-scaled GEMM wants its 128-row tiles on
// 128-row boundaries of the sorted buffer: the scale atoms are 128 rows tall); rows_out then counts the gaps too.
__device__ __forceinline__ void moe_plan_body(const int* topk_ids, int* perm, int* offsets, int* tiles, int* tile_count,
                                              int* rows_out, int entries, int e_lo, int e_hi, int bm, int max_tiles, int* err,
                                              int rank, int per_rank, int align, int k = 1, int* src_tok = nullptr,
                                              int* row_choice = nullptr, int max_rows = 0) {
  pdl_wait();
  // the inverse of perm for the expert-parallel kernels: the token and the choice of every sorted row, -1 in the gaps
  if (src_tok != nullptr)
    for (int i = threadIdx.x; i < max_rows; i += blockDim.x) src_tok[i] = -1;
  e_lo += rank * per_rank;      // expert parallel: rank r keeps experts [e_lo + r * per_rank, e_hi + r * per_rank)
  e_hi += rank * per_rank;
  extern __shared__ int sm[];          // counts[E_local] | cursor[E_local]
  const int el = e_hi - e_lo;
  int* counts = sm;
  int* cursor = sm + el;
  for (int i = threadIdx.x; i < el; i += blockDim.x) counts[i] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < entries; i += blockDim.x) {
    const int e = topk_ids[i];
    if (e >= e_lo && e < e_hi) atomicAdd(&counts[e - e_lo], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, nt = 0;
    for (int e = 0; e < el; ++e) {
      if (align > 1 && counts[e] > 0) at = (at + align - 1) / align * align;
      offsets[e] = at;
      cursor[e] = at;
      for (int m0 = 0; m0 < counts[e]; m0 += bm) {
        if (nt < max_tiles) {
          reinterpret_cast<int4*>(tiles)[nt] = make_int4(e, at + m0, min(bm, counts[e] - m0), 0);
          ++nt;
        } else {
          set_error(err, ERR_BOUNDS);
        }
      }
      at += counts[e];
    }
    offsets[el] = at;
    tile_count[0] = nt;
    rows_out[0] = at;
  }
  __syncthreads();
  // placement: an entry takes the next free row of its expert. The order inside an expert is whatever the atomics
  // give; every output row depends only on its own input row and the expert's weights, so the result's bits do not.
  for (int i = threadIdx.x; i < entries; i += blockDim.x) {
    const int e = topk_ids[i];
    const int r = (e >= e_lo && e < e_hi) ? atomicAdd(&cursor[e - e_lo], 1) : -1;
    perm[i] = r;
    if (src_tok != nullptr && r >= 0) {
      if (r < max_rows) {
        src_tok[r] = i / k;
        row_choice[r] = i % k;
      } else {
        set_error(err, ERR_BOUNDS);
      }
    }
  }
}

extern "C" __global__ void __launch_bounds__(1024)
    kern_moe_plan(const int* topk_ids, int* perm, int* offsets, int* tiles, int* tile_count, int* rows_out, int entries,
                  int e_lo, int e_hi, int bm, int max_tiles, int* err, int rank, int per_rank) {
  moe_plan_body(topk_ids, perm, offsets, tiles, tile_count, rows_out, entries, e_lo, e_hi, bm, max_tiles, err, rank, per_rank, 1);
}
extern "C" __global__ void __launch_bounds__(1024)
    kern_moe_plan_aligned(const int* topk_ids, int* perm, int* offsets, int* tiles, int* tile_count, int* rows_out,
                          int entries, int e_lo, int e_hi, int bm, int max_tiles, int* err, int rank, int per_rank) {
  moe_plan_body(topk_ids, perm, offsets, tiles, tile_count, rows_out, entries, e_lo, e_hi, bm, max_tiles, err, rank, per_rank, bm);
}

// grid = entries (tokens * k), block 128; 16-byte vectors.
extern "C" __global__ void __launch_bounds__(128)
    kern_moe_gather_bf16(const __nv_bfloat16* x, const int* perm, __nv_bfloat16* x_perm, int entries, int k, int hidden) {
  pdl_wait();
  const int i = blockIdx.x;
  if (i >= entries) return;
  const int r = perm[i];
  if (r < 0) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(i / k) * hidden);
  uint4* dst = reinterpret_cast<uint4*>(x_perm + (size_t)r * hidden);
  if (!KERN_CHECK(dst, (size_t)hidden * 2, SITE_MOE_GATHER)) return;
  for (int v = threadIdx.x; v < hidden / 8; v += 128) dst[v] = src[v];
}

// grid = tokens, block 128. out may alias shared (read before write per element).
extern "C" __global__ void __launch_bounds__(128)
    kern_moe_combine_bf16(const __nv_bfloat16* y_perm, const int* perm, const float* topk_w, const __nv_bfloat16* shared,
                          __nv_bfloat16* out, int tokens, int k, int hidden, int accumulate) {
  pdl_wait();
  const int t = blockIdx.x;
  if (t >= tokens) return;
  for (int v = threadIdx.x; v < hidden / 8; v += 128) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    auto add = [&](uint4 p, float w) {
      float2 a = unpack_bf16x2(p.x), b = unpack_bf16x2(p.y), c = unpack_bf16x2(p.z), d = unpack_bf16x2(p.w);
      acc[0] += w * a.x; acc[1] += w * a.y; acc[2] += w * b.x; acc[3] += w * b.y;
      acc[4] += w * c.x; acc[5] += w * c.y; acc[6] += w * d.x; acc[7] += w * d.y;
    };
    if (accumulate) add(reinterpret_cast<const uint4*>(out + (size_t)t * hidden)[v], 1.f);
    if (shared) add(reinterpret_cast<const uint4*>(shared + (size_t)t * hidden)[v], 1.f);
    for (int j = 0; j < k; ++j) {
      const int r = perm[(size_t)t * k + j];
      if (r >= 0 && KERN_CHECK(y_perm + (size_t)r * hidden, (size_t)hidden * 2, SITE_MOE_COMBINE))
        add(reinterpret_cast<const uint4*>(y_perm + (size_t)r * hidden)[v], topk_w[(size_t)t * k + j]);
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out + (size_t)t * hidden)[v] = o;
  }
}

#define KERN_MOE_GEMM_ENTRY(name, BN, EPI)                                                                        \
  extern "C" __global__ void __launch_bounds__(192, 1)                                                            \
      name(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, void* C,          \
           const int* tiles, const int* tile_count, int M, int N, int K, int ldc, int* err) {                      \
    kern::gemm_body<BN, EPI, true>(&tma_a, &tma_b, C, nullptr, M, N, K, ldc, err, tiles, tile_count);              \
  }

KERN_MOE_GEMM_ENTRY(kern_moe_gemm_bf16_n256, 256, 0)
KERN_MOE_GEMM_ENTRY(kern_moe_gemm_bf16_n128, 128, 0)
KERN_MOE_GEMM_ENTRY(kern_moe_gemm_bf16_n64, 64, 0)
KERN_MOE_GEMM_ENTRY(kern_moe_gemm_bf16_swiglu_n256, 256, 3)
KERN_MOE_GEMM_ENTRY(kern_moe_gemm_bf16_swiglu_n128, 128, 3)
KERN_MOE_GEMM_ENTRY(kern_moe_gemm_bf16_swiglu_n64, 64, 3)

// ---- expert parallel over sharded tokens: dispatch by pull, combine by push -------------------------------------------
// Tokens live on their home rank (rows_per_rank each, token t = home * rows_per_rank + local row); every rank knows
// every token's expert choices (an all-gather of the ids) and plans over all of them, keeping the entries of its own
// experts. The gather below IS the dispatch: it reads exactly the rows this rank's experts need, straight out of the
// home ranks' exported activation buffers (16-byte peer loads, several in flight per thread). After the grouped GEMMs,
// the return kernel pushes every result row into slot (local row, choice) of the home rank's exported return buffer
// (plain 16-byte peer stores; a slot has exactly one writer), and the home rank's combine weighs its k slots.
// Barriers (kern_peer_barrier) stand before the pull and after the push.
// Reference counterpart: docs/roadmap.md:13-16,63 (all-to-all / all-gather -> FC1 -> FC2 -> finalize -> reduce-scatter).

// grid = entries (tokens * k), block 128.
extern "C" __global__ void __launch_bounds__(128)
    kern_moe_gather_peers_bf16(const unsigned long long* x_peers, const int* perm, __nv_bfloat16* x_perm, int entries, int k,
                               int hidden, int rows_per_rank) {
  pdl_wait();
  const int i = blockIdx.x;
  if (i >= entries) return;
  const int r = perm[i];
  if (r < 0) return;
  const int t = i / k;
  const uint8_t* src = reinterpret_cast<const uint8_t*>(x_peers[t / rows_per_rank]) + (size_t)(t % rows_per_rank) * hidden * 2;
  uint4* dst = reinterpret_cast<uint4*>(x_perm + (size_t)r * hidden);
  if (!KERN_CHECK(src, (size_t)hidden * 2, SITE_EP_PULL) || !KERN_CHECK(dst, (size_t)hidden * 2, SITE_MOE_GATHER)) return;
  const int vecs = hidden / 8;
  for (int v0 = threadIdx.x; v0 < vecs; v0 += 128 * 4) {
    uint4 x[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int v = v0 + u * 128;
      if (v < vecs)
        asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(x[u].x), "=r"(x[u].y), "=r"(x[u].z), "=r"(x[u].w) : "l"(src + (size_t)v * 16));
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int v = v0 + u * 128;
      if (v < vecs) dst[v] = x[u];
    }
  }
}

// grid = entries, block 128: y_perm[perm[i]] -> ret of the home rank, slot (local row, choice).
extern "C" __global__ void __launch_bounds__(128)
    kern_moe_return_bf16(const __nv_bfloat16* y_perm, const int* perm, const unsigned long long* ret_peers, int entries, int k,
                         int hidden, int rows_per_rank) {
  pdl_wait();
  const int i = blockIdx.x;
  if (i >= entries) return;
  const int r = perm[i];
  if (r < 0) return;
  const int t = i / k, j = i % k;
  uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(ret_peers[t / rows_per_rank]) +
                                        ((size_t)(t % rows_per_rank) * k + j) * hidden * 2);
  const uint4* src = reinterpret_cast<const uint4*>(y_perm + (size_t)r * hidden);
  if (!KERN_CHECK(dst, (size_t)hidden * 2, SITE_EP_SLOT) || !KERN_CHECK(src, (size_t)hidden * 2, SITE_MOE_COMBINE)) return;
  for (int v = threadIdx.x; v < hidden / 8; v += 128) dst[v] = src[v];
}

// ---- expert parallel over sharded tokens, fused: dispatch inside FC1, combine inside FC2 ------------------------------
// Per layer and rank, five launches and no barrier kernel, no NCCL call:
//   kern_ep_publish      this rank's expert ids into every rank's table (peer stores), then its epoch into every rank's
//                        `ids_ready` words
//   kern_moe_plan_ep     waits (bounded) until every rank's ids of this epoch are here, then plans over all tokens for
//                        this rank's experts: tile table on 128-row boundaries, token and choice of every sorted row
//   kern_ep_fc1_*        routed GEMM + SwiGLU whose gather warps pull the rows out of the home ranks while tiles run (EP 1)
//   kern_ep_fc2_*        routed GEMM whose epilogue stores every result row into its (token, choice) slot on the token's
//                        home rank and publishes `done` when the grid has finished (EPI 5)
//   kern_ep_finalize     waits (bounded) for every rank's `done`, then out[t] = sum_j w[t, j] * slot[t, j] (plus an optional
//                        shared-expert / residual term): the top-k weighted reduction, on the home rank
// Hazards are closed by the two flag rounds: a rank rewrites its activations or ids only after its finalize, which has
// seen every peer's FC2 - and therefore its plan and its pulls - finished; a peer writes a slot only after its plan has
// seen the home rank's publish, which is after the home rank's previous finalize (the slots' reader) in stream order.
// Reference: docs/roadmap.md:13-16 (one-launch routed layer), docs/runtime.md:201-202, crates/kern-runtime/src/nccl.rs:238-256
// (the all-to-all the reference's un-fused path uses).

// One CTA. grid = 1, block 1024.
extern "C" __global__ void __launch_bounds__(1024)
    kern_ep_publish(const int* ids, const unsigned long long* ids_peers, const unsigned long long* ready_peers,
                    uint32_t* epoch, int tokens, int rows_per_rank, int k, int rank, int nranks) {
  pdl_wait();
  const int n = rows_per_rank * k, have = tokens * k;
  for (int r = 0; r < nranks; ++r) {
    int* di = reinterpret_cast<int*>(ids_peers[r]) + (size_t)rank * n;
    for (int i = threadIdx.x; i < n; i += blockDim.x) di[i] = i < have ? ids[i] : -1;   // rows not in this step route nowhere
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t e = epoch[0] + 1;
    epoch[0] = e;
    for (int r = 0; r < nranks; ++r) st_release_sys(reinterpret_cast<uint32_t*>(ready_peers[r]) + rank, e);
  }
}

extern "C" __global__ void __launch_bounds__(1024)
    kern_moe_plan_ep(const int* ids_all, int* perm, int* offsets, int* tiles, int* tile_count, int* rows_out, int* src_tok,
                     int* row_choice, const uint32_t* ready, const uint32_t* epoch, int entries, int k, int e_n, int bm,
                     int max_tiles, int max_rows, int* err, int rank, int nranks, long long timeout_ns) {
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  if ((int)threadIdx.x < nranks) {
    const uint32_t e = epoch[0];
    const uint64_t t0 = globaltimer_ns();
    while ((int32_t)(ld_acquire_sys(ready + threadIdx.x) - e) < 0) {
      if ((long long)(globaltimer_ns() - t0) > timeout_ns) {
        set_error(err, ERR_WAIT_PEER + threadIdx.x);
        failed = 1;
        break;
      }
      __nanosleep(40);
    }
  }
  __syncthreads();
  if (failed) {                      // no plan: the routed GEMMs see zero tiles
    if (threadIdx.x == 0) { tile_count[0] = 0; rows_out[0] = 0; }
    return;
  }
  moe_plan_body(ids_all, perm, offsets, tiles, tile_count, rows_out, entries, 0, e_n, bm, max_tiles, err, rank, e_n, bm, k,
                src_tok, row_choice, max_rows);
}

#define KERN_EP_FC1_ENTRY(name, BN)                                                                                    \
  extern "C" __global__ void __launch_bounds__(320, 1)                                                                 \
      name(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, void* C,               \
           const int* tiles, const int* tile_count, int M, int N, int K, int ldc, int* err,                             \
           const unsigned long long* x_peers, __nv_bfloat16* xg, const int* src_tok, uint32_t* flags,                   \
           uint32_t* cta_epochs, int rows_per_rank, int max_blocks, int rank, int nranks) {                             \
    kern::AgArgs ag;                                                                                                   \
    ag.flags = flags; ag.epochs = cta_epochs; ag.max_blocks = max_blocks; ag.rank = rank; ag.nranks = nranks;          \
    kern::EpArgs ep;                                                                                                   \
    ep.x_peers = x_peers; ep.xg = xg; ep.src_tok = src_tok; ep.rows_per_rank = rows_per_rank;                          \
    if (*tile_count > max_blocks) { /* every 128-row block needs its counter */                                        \
      if (threadIdx.x == 0 && blockIdx.x == 0) kern::set_error(err, kern::ERR_BOUNDS);                                 \
      return;                                                                                                          \
    }                                                                                                                  \
    kern::gemm_body<BN, 3, true, false, false, true, 1>(&tma_a, &tma_b, C, nullptr, M, N, K, ldc, err, tiles,          \
                                                        tile_count, kern::ScatterArgs(), nullptr, nullptr, ag, ep);    \
  }

KERN_EP_FC1_ENTRY(kern_ep_fc1_bf16_swiglu_n256, 256)
KERN_EP_FC1_ENTRY(kern_ep_fc1_bf16_swiglu_n128, 128)
KERN_EP_FC1_ENTRY(kern_ep_fc1_bf16_swiglu_n64, 64)

#define KERN_EP_FC2_ENTRY(name, BN)                                                                                    \
  extern "C" __global__ void __launch_bounds__(192, 1)                                                                 \
      name(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const int* tiles,      \
           const int* tile_count, int M, int N, int K, int* err, const unsigned long long* ret_peers,                   \
           const int* src_tok, const int* row_choice, uint32_t* state, const unsigned long long* done_peers,            \
           int rows_per_rank, int k, int rank, int nranks) {                                                           \
    kern::EpArgs ep;                                                                                                   \
    ep.ret_peers = ret_peers; ep.src_tok = src_tok; ep.row_choice = row_choice; ep.state = state;                      \
    ep.done_peers = done_peers; ep.rows_per_rank = rows_per_rank; ep.k = k; ep.rank = rank; ep.nranks = nranks;        \
    kern::gemm_body<BN, 5, true>(&tma_a, &tma_b, nullptr, nullptr, M, N, K, N, err, tiles, tile_count,                 \
                                 kern::ScatterArgs(), nullptr, nullptr, kern::AgArgs(), ep);                          \
  }

KERN_EP_FC2_ENTRY(kern_ep_fc2_bf16_combine_n256, 256)
KERN_EP_FC2_ENTRY(kern_ep_fc2_bf16_combine_n128, 128)
KERN_EP_FC2_ENTRY(kern_ep_fc2_bf16_combine_n64, 64)

// grid = this rank's tokens, block 128. out[t] = sum_j w[t, j] * ret[t, j] (+ out[t] when accumulate) (+ extra[t]).
extern "C" __global__ void __launch_bounds__(128)
    kern_ep_finalize(const __nv_bfloat16* ret, const float* topk_w, __nv_bfloat16* out, const __nv_bfloat16* extra,
                     const uint32_t* done, const uint32_t* state, int* err, int tokens, int k, int hidden, int nranks,
                     long long timeout_ns, int accumulate) {
  pdl_wait();
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  if ((int)threadIdx.x < nranks) {
    const uint32_t e = state[1];
    const uint64_t t0 = globaltimer_ns();
    while ((int32_t)(ld_acquire_sys(done + threadIdx.x) - e) < 0) {
      if ((long long)(globaltimer_ns() - t0) > timeout_ns) {
        set_error(err, ERR_WAIT_PEER + threadIdx.x);
        failed = 1;
        break;
      }
      __nanosleep(40);
    }
  }
  __syncthreads();
  if (failed) return;
  const int t = blockIdx.x;
  if (t >= tokens) return;
  for (int v = threadIdx.x; v < hidden / 8; v += 128) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    auto add = [&](uint4 p, float w) {
      float2 a = unpack_bf16x2(p.x), b = unpack_bf16x2(p.y), c = unpack_bf16x2(p.z), d = unpack_bf16x2(p.w);
      acc[0] += w * a.x; acc[1] += w * a.y; acc[2] += w * b.x; acc[3] += w * b.y;
      acc[4] += w * c.x; acc[5] += w * c.y; acc[6] += w * d.x; acc[7] += w * d.y;
    };
    if (accumulate) add(reinterpret_cast<const uint4*>(out + (size_t)t * hidden)[v], 1.f);
    if (extra != nullptr) add(reinterpret_cast<const uint4*>(extra + (size_t)t * hidden)[v], 1.f);
    for (int j = 0; j < k; ++j) {
      // the slots were written by other GPUs: read them past this SM's L1
      uint4 p;
      const uint4* src = reinterpret_cast<const uint4*>(ret + ((size_t)t * k + j) * hidden) + v;
      asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(p.x), "=r"(p.y), "=r"(p.z), "=r"(p.w) : "l"(src));
      add(p, topk_w[(size_t)t * k + j]);
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out + (size_t)t * hidden)[v] = o;
  }
}
