// Gated DeltaNet (linear attention with a gated delta rule) for hybrid decoders: causal short
// convolution + SiLU over the q|k|v channels, and the recurrent state update, for decode rows and for
// ragged prefill chunks. One per-sequence state line per layer:
//     [conv window: (width-1) x conv_dim bf16][S: HV x DV x DK f32]
// line 0 is the null line (padding rows use it and nothing is written to it).
//
// Per (sequence, value head hv), per token:
//   q = l2norm(q) / sqrt(DK);  k = l2norm(k);  g = -exp(A_log[hv]) * softplus(a + dt_bias[hv]);  beta = sigmoid(b)
//   S *= exp(g);  u = (v - S k) * beta;  S += u k^T;  o = S q;  y = rmsnorm(o) * w * silu(z)
// Reference counterpart: tools/kernels-src/gdn_decode.cu:90 (conv), :171 (step) — decode only; the
// reference takes chunked prefill as a mined kernel. Here one kernel body serves both: a CTA keeps its
// sixteen state rows in registers for the whole chunk of a sequence and walks the tokens in order.
#include "common.cuh"

using namespace kern;

// ---- causal conv (width <= 4) + SiLU ----------------------------------------------------------------
// x: [tokens][x_stride] (the q|k|v channels are the first conv_dim of a row), y: [tokens][conv_dim]
// w: [conv_dim][width] bf16, bias optional. cu_q: [seqs+1] row starts (nullptr: one row per sequence).
// Every output row depends on at most width-1 earlier inputs, so rows are independent: grid
// [ceil(rows / rpc), ceil(conv_dim / 1024)], block 256; a thread owns four adjacent channels (8-byte loads and stores;
// conv_dim is a multiple of 4) and walks rpc consecutive rows (16 for prefill chunks, 1 for decode rows),
// carrying the last inputs in registers and re-seeding them from the state window at a sequence's first row.
// The window itself is advanced afterwards by kern_gdn_conv_state (a separate launch: rows of one sequence may sit
// in several CTAs, and none of them may see the window half-updated).
extern "C" __global__ void __launch_bounds__(256)
    kern_gdn_conv_bf16(const __nv_bfloat16* x, __nv_bfloat16* y, const uint8_t* state, const int* lines, const int* cu_q,
                       const __nv_bfloat16* w, const __nv_bfloat16* bias, int seqs, int rows, int conv_dim, int width,
                       int x_stride, long long line_bytes, int rpc) {
  pdl_wait();
  const int c = (blockIdx.y * 256 + threadIdx.x) * 4;
  const int total = cu_q ? min(rows, cu_q[seqs]) : min(rows, seqs);
  const int ra = blockIdx.x * rpc, rb = min(total, ra + rpc);
  if (c >= conv_dim || ra >= rb) return;
  auto load4 = [](const __nv_bfloat16* p, float (&o)[4]) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
    o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
  };
  float wt[4][4];      // [channel][tap], right-aligned: tap 3 multiplies the current row, tap 2 the row before, ...
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) wt[i][j] = j >= 4 - width ? __bfloat162float(w[(size_t)(c + i) * width + j - (4 - width)]) : 0.f;
  float bs[4] = {0.f, 0.f, 0.f, 0.f};
  if (bias) load4(bias + c, bs);
  // the sequence of row ra: the last s with cu_q[s] <= ra
  int s = ra;
  if (cu_q) {
    int lo = 0, hi = seqs - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (cu_q[mid] <= ra) lo = mid; else hi = mid - 1;
    }
    s = lo;
  }
  int r0 = cu_q ? cu_q[s] : s, r1 = cu_q ? cu_q[s + 1] : s + 1;
  float hist[3][4];     // inputs r-3, r-2, r-1 (only the last width-1 matter)
#pragma unroll
  for (int d = 0; d < 3; ++d)
#pragma unroll
    for (int i = 0; i < 4; ++i) hist[d][i] = 0.f;
  auto seed = [&](int r) {
    int line = lines[s];
  if (line > 0 && !KERN_CHECK(state + (size_t)line * line_bytes, (size_t)line_bytes, SITE_STATE_SLOT)) line = 0;   // checked builds: a slot outside the pool is the null line
    const __nv_bfloat16* win = reinterpret_cast<const __nv_bfloat16*>(state + (size_t)line * line_bytes);
#pragma unroll
    for (int d = 1; d <= 3; ++d) {
      if (d > width - 1) continue;
      const int rr = r - d;
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      if (rr >= r0) load4(x + (size_t)rr * x_stride + c, v);
      else if (line > 0) load4(win + (size_t)(width - 1 - (r0 - rr)) * conv_dim + c, v);
#pragma unroll
      for (int i = 0; i < 4; ++i) hist[3 - d][i] = v[i];
    }
  };
  seed(ra);
  for (int r = ra; r < rb; ++r) {
    while (r >= r1) {     // next sequence (empty ones are skipped)
      ++s;
      r0 = cu_q ? cu_q[s] : s;
      r1 = cu_q ? cu_q[s + 1] : s + 1;
      if (r < r1) seed(r);
    }
    float cur[4], o[4];
    load4(x + (size_t)r * x_stride + c, cur);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float acc = bs[i] + wt[i][3] * cur[i] + wt[i][2] * hist[2][i] + wt[i][1] * hist[1][i] + wt[i][0] * hist[0][i];
      o[i] = silu(acc);
      hist[0][i] = hist[1][i]; hist[1][i] = hist[2][i]; hist[2][i] = cur[i];
    }
    *reinterpret_cast<uint2*>(y + (size_t)r * conv_dim + c) = make_uint2(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]));
  }
}

// One row per sequence (decode): the conv of the row and the shift of its window in ONE launch — a thread owns four
// channels of one sequence, so it reads its own window, writes y, and then writes the shifted window; nobody else
// touches those bytes. grid [seqs, ceil(conv_dim / 1024)], block 256. Row s belongs to sequence s.
extern "C" __global__ void __launch_bounds__(256)
    kern_gdn_conv_step_bf16(const __nv_bfloat16* x, __nv_bfloat16* y, uint8_t* state, const int* lines, const __nv_bfloat16* w,
                            const __nv_bfloat16* bias, int seqs, int conv_dim, int width, int x_stride, long long line_bytes) {
  pdl_wait();
  const int s = blockIdx.x;
  const int c = (blockIdx.y * 256 + threadIdx.x) * 4;
  if (s >= seqs || c >= conv_dim) return;
  auto load4 = [](const __nv_bfloat16* p, float (&o)[4]) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
    o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
  };
  int line = lines[s];
  if (line > 0 && !KERN_CHECK(state + (size_t)line * line_bytes, (size_t)line_bytes, SITE_STATE_SLOT)) line = 0;   // checked builds: a slot outside the pool is the null line
  const int keep = width - 1;
  __nv_bfloat16* win = reinterpret_cast<__nv_bfloat16*>(state + (size_t)line * line_bytes);
  float hist[3][4];        // right-aligned: hist[2] is the previous row
  uint2 raw[3];
#pragma unroll
  for (int d = 0; d < 3; ++d) {
    raw[d] = make_uint2(0u, 0u);
#pragma unroll
    for (int i = 0; i < 4; ++i) hist[d][i] = 0.f;
  }
#pragma unroll
  for (int d = 0; d < 3; ++d) {
    if (d < 3 - keep || line <= 0) continue;                    // window row d - (3 - keep)
    raw[d] = *reinterpret_cast<const uint2*>(win + (size_t)(d - (3 - keep)) * conv_dim + c);
    const float2 a = unpack_bf16x2(raw[d].x), b = unpack_bf16x2(raw[d].y);
    hist[d][0] = a.x; hist[d][1] = a.y; hist[d][2] = b.x; hist[d][3] = b.y;
  }
  float cur[4], bs[4] = {0.f, 0.f, 0.f, 0.f}, o[4];
  const uint2 xr = *reinterpret_cast<const uint2*>(x + (size_t)s * x_stride + c);
  load4(x + (size_t)s * x_stride + c, cur);
  if (bias) load4(bias + c, bs);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float wt[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) wt[j] = j >= 4 - width ? __bfloat162float(w[(size_t)(c + i) * width + j - (4 - width)]) : 0.f;
    o[i] = silu(bs[i] + wt[3] * cur[i] + wt[2] * hist[2][i] + wt[1] * hist[1][i] + wt[0] * hist[0][i]);
  }
  *reinterpret_cast<uint2*>(y + (size_t)s * conv_dim + c) = make_uint2(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]));
  if (line > 0) {
    // new window = old rows 1 .. keep-1, then this row
#pragma unroll
    for (int d = 0; d < 3; ++d) {
      if (d < 3 - keep) continue;
      const int j = d - (3 - keep);                                // window row j takes old row j + 1, the last one x
      *reinterpret_cast<uint2*>(win + (size_t)j * conv_dim + c) = d == 2 ? xr : raw[d + 1];
    }
  }
}

// window' = the last width-1 inputs of (window ++ this call's rows). grid [seqs, ceil(conv_dim / 256)], block 256.
extern "C" __global__ void __launch_bounds__(256)
    kern_gdn_conv_state(const __nv_bfloat16* x, uint8_t* state, const int* lines, const int* cu_q, int seqs, int conv_dim,
                        int width, int x_stride, long long line_bytes) {
  pdl_wait();
  const int s = blockIdx.x;
  const int c = blockIdx.y * 256 + threadIdx.x;
  if (s >= seqs || c >= conv_dim) return;
  int line = lines[s];
  if (line > 0 && !KERN_CHECK(state + (size_t)line * line_bytes, (size_t)line_bytes, SITE_STATE_SLOT)) line = 0;   // checked builds: a slot outside the pool is the null line
  const int r0 = cu_q ? cu_q[s] : s, r1 = cu_q ? cu_q[s + 1] : s + 1;
  const int n = r1 - r0, keep = width - 1;
  if (line <= 0 || n <= 0) return;
  __nv_bfloat16* win = reinterpret_cast<__nv_bfloat16*>(state + (size_t)line * line_bytes);
  __nv_bfloat16 nw[3];
  for (int j = 0; j < keep; ++j) {
    const int src = n + j - keep;      // index into this call's rows; negative: still in the old window
    nw[j] = src >= 0 ? x[(size_t)(r0 + src) * x_stride + c] : win[(size_t)(keep + src) * conv_dim + c];
  }
  for (int j = 0; j < keep; ++j) win[(size_t)j * conv_dim + c] = nw[j];
}

// ---- gated delta rule ---------------------------------------------------------------------------------
// qkv: conv output [tokens][conv_dim] laid out [q: HK*DK | k: HK*DK | v: HV*DV]
// zba: [tokens][zba_stride] with b at b_off (HV), a at a_off (HV)   (bf16)
// o_raw: [tokens][HV*DV] f32, the un-normalised output S q (kern_gdn_gate_norm_bf16 finishes it).
// A_log, dt_bias: f32 [HV].
//
// Every value row of S has its own recurrence (u[v] = beta (v[v] - S[v,:] k); S[v,:] += u[v] k), so a head is
// split over DV / 16 CTAs of 16 rows each: grid [HV * DV/16, seqs], block 256. Sixteen lanes share a row, each
// keeping DK/16 state elements in registers for the whole chunk of the sequence: the token loop touches no
// shared-memory state and has no block barrier, only two 16-lane shuffle reductions per token. Tokens are
// staged 32 at a time: q and k are loaded, l2-normalised (one warp per token) and parked in shared memory
// together with v, the decay and beta of those tokens.
constexpr int GDN_TB = 32;     // most tokens per staged batch

template <int DK, int DV, int ROWS, bool KDA = false>   // ROWS value rows per CTA. 16 everywhere: 64 rows per CTA pay the staged q/k reads and
                                      // the shuffles once per 64 rows, but leave 96 CTAs of 8 warps on 148 SMs and measured
                                      // slower (1.44 ms against 1.27 ms per 2048-row chunk)
__device__ __forceinline__ void gdn_body(const __nv_bfloat16* qkv, const __nv_bfloat16* zba, float* o_raw, uint8_t* state,
                                         const int* lines, const int* cu_q, const float* A_log, const float* dt_bias,
                                         int seqs, int hk, int hv, int zba_stride, int b_off, int a_off,
                                         long long line_bytes, long long s_offset, int tb,
                                         const __nv_bfloat16* gk = nullptr, int gk_stride = 0) {
  constexpr int TPR = 256 / ROWS;       // lanes per value row
  constexpr int KPT = DK / TPR;         // state elements per thread, in 16-byte groups: group g of a thread is keys
                                        // g * 4 TPR + part * 4 .. + 3, so a row's 16 lanes read 256 contiguous bytes per access
  constexpr int VEC = KPT % 4 == 0 ? 4 : KPT;      // elements per group (DK = 32: one 8-byte group)
  constexpr int NG = KPT / VEC;
  static_assert(KPT >= 1 && DV % ROWS == 0 && TPR <= 32, "shape");
  // staging for `tb` tokens (dynamic shared memory: (2 DK + ROWS + 4) * 4 bytes per token) — a decode launch stages
  // one token and leaves the SM's shared memory to more resident CTAs.  meta[t] = {decay, beta, k.q, -}
  extern __shared__ __align__(16) float gdn_sm[];
  float (*qs)[DK] = reinterpret_cast<float (*)[DK]>(gdn_sm);
  float (*ks)[DK] = reinterpret_cast<float (*)[DK]>(gdn_sm + (size_t)tb * DK);
  float4* meta = reinterpret_cast<float4*>(gdn_sm + (size_t)2 * tb * DK);
  float (*vs)[ROWS] = reinterpret_cast<float (*)[ROWS]>(gdn_sm + (size_t)tb * (2 * DK + 4));
  float (*ds)[DK] = reinterpret_cast<float (*)[DK]>(gdn_sm + (size_t)tb * (2 * DK + 4 + ROWS));     // KDA: decay per key
  constexpr int PARTS = DV / ROWS;
  const int h = blockIdx.x / PARTS, row0 = (blockIdx.x % PARTS) * ROWS, s = blockIdx.y;
  if (s >= seqs) return;
  int line = lines[s];
  if (line > 0 && !KERN_CHECK(state + (size_t)line * line_bytes, (size_t)line_bytes, SITE_STATE_SLOT)) line = 0;   // checked builds: a slot outside the pool is the null line
  const int r0 = cu_q ? cu_q[s] : s, r1 = cu_q ? cu_q[s + 1] : s + 1;
  if (r1 <= r0) return;
  const int kh = h / (hv / hk);
  const int conv_dim = 2 * hk * DK + hv * DV;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int vrow = tid / TPR, kpart = tid % TPR;
  float* Sg = reinterpret_cast<float*>(state + (size_t)line * line_bytes + s_offset) +
              ((size_t)h * DV + row0 + vrow) * DK;
  auto kidx = [&](int j) { return (j / VEC) * (VEC * TPR) + kpart * VEC + (j % VEC); };
  float S[KPT];
  if constexpr (VEC == 4) {
#pragma unroll
    for (int g = 0; g < NG; ++g) {
      const float4 v = line > 0 ? *reinterpret_cast<const float4*>(Sg + g * 4 * TPR + kpart * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
      S[4 * g] = v.x; S[4 * g + 1] = v.y; S[4 * g + 2] = v.z; S[4 * g + 3] = v.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < KPT; ++j) S[j] = line > 0 ? Sg[kidx(j)] : 0.f;
  }
  const float a_neg = -__expf(A_log[h]);
  const float dtb = dt_bias[h];
  constexpr int QN = (DK + 31) / 32;
  for (int base = r0; base < r1; base += tb) {
    const int nb = min(tb, r1 - base);
    __syncthreads();   // the previous batch has been consumed
    // a warp stages tokens warp, warp + 8, ...: all their loads are issued first, then each is normalised and parked
    float pq[GDN_TB / 8][QN], pk[GDN_TB / 8][QN];
#pragma unroll
    for (int u = 0; u < GDN_TB / 8; ++u) {
      const int t = warp + u * 8;
      if (t < nb) {
        const __nv_bfloat16* row = qkv + (size_t)(base + t) * conv_dim;
#pragma unroll
        for (int i = 0; i < QN; ++i) {
          const int c = i * 32 + lane;
          pq[u][i] = c < DK ? __bfloat162float(row[kh * DK + c]) : 0.f;
          pk[u][i] = c < DK ? __bfloat162float(row[hk * DK + kh * DK + c]) : 0.f;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < GDN_TB / 8; ++u) {
      const int t = warp + u * 8;
      if (t < nb) {
        const __nv_bfloat16* row = qkv + (size_t)(base + t) * conv_dim;
        float q2 = 0.f, k2 = 0.f, qk = 0.f;
#pragma unroll
        for (int i = 0; i < QN; ++i) { q2 += pq[u][i] * pq[u][i]; k2 += pk[u][i] * pk[u][i]; qk += pq[u][i] * pk[u][i]; }
        q2 = warp_sum(q2);
        k2 = warp_sum(k2);
        qk = warp_sum(qk);
        const float qi = rsqrtf(q2 + 1e-6f) * rsqrtf((float)DK), ki = rsqrtf(k2 + 1e-6f);
#pragma unroll
        for (int i = 0; i < QN; ++i) {
          const int c = i * 32 + lane;
          if (c < DK) {
            qs[t][c] = pq[u][i] * qi;
            ks[t][c] = pk[u][i] * ki;
            if constexpr (KDA) {
              const float x = __bfloat162float(gk[(size_t)(base + t) * gk_stride + h * DK + c]) + dt_bias[h * DK + c];
              ds[t][c] = __expf(a_neg * (x > 20.f ? x : log1pf(__expf(x))));
            }
          }
        }
        for (int r = lane; r < ROWS; r += 32) vs[t][r] = __bfloat162float(row[2 * hk * DK + h * DV + row0 + r]);
        if (lane == 31) {
          const float av = __bfloat162float(zba[(size_t)(base + t) * zba_stride + a_off + h]) + dtb;
          const float sp = av > 20.f ? av : log1pf(__expf(av));
          const float bb = __bfloat162float(zba[(size_t)(base + t) * zba_stride + b_off + h]);
          meta[t] = make_float4(__expf(a_neg * sp), __bfloat162float(__float2bfloat16(1.f / (1.f + __expf(-bb)))),
                                qk * qi * ki, 0.f);
        }
      }
    }
    __syncthreads();
    for (int t = 0; t < nb; ++t) {
      const float4 m = meta[t];            // decay, beta, k.q
      const float vv = vs[t][vrow];
      float kr[KPT], qr[KPT];
      if constexpr (VEC == 4) {
#pragma unroll
        for (int j = 0; j < NG; ++j) {
          const float4 k4 = *reinterpret_cast<const float4*>(&ks[t][j * 4 * TPR + kpart * 4]);
          const float4 q4 = *reinterpret_cast<const float4*>(&qs[t][j * 4 * TPR + kpart * 4]);
          kr[4 * j] = k4.x; kr[4 * j + 1] = k4.y; kr[4 * j + 2] = k4.z; kr[4 * j + 3] = k4.w;
          qr[4 * j] = q4.x; qr[4 * j + 1] = q4.y; qr[4 * j + 2] = q4.z; qr[4 * j + 3] = q4.w;
        }
      } else {
#pragma unroll
        for (int j = 0; j < KPT; ++j) { kr[j] = ks[t][kidx(j)]; qr[j] = qs[t][kidx(j)]; }
      }
      // both products run on the state *before* this token: S_t q = decay (S_{t-1} q) + u (k.q), so one round of
      // shuffles carries the two sums instead of two rounds in sequence
      if constexpr (KDA) {      // decay per key channel, applied before both products
        if constexpr (VEC == 4) {
#pragma unroll
          for (int j = 0; j < NG; ++j) {
            const float4 d4 = *reinterpret_cast<const float4*>(&ds[t][j * 4 * TPR + kpart * 4]);
            S[4 * j] *= d4.x; S[4 * j + 1] *= d4.y; S[4 * j + 2] *= d4.z; S[4 * j + 3] *= d4.w;
          }
        } else {
#pragma unroll
          for (int j = 0; j < KPT; ++j) S[j] *= ds[t][kidx(j)];
        }
      }
      const float dcy = KDA ? 1.f : m.x;
      float sa = 0.f, sb = 0.f;
#pragma unroll
      for (int j = 0; j < KPT; ++j) { sa += S[j] * kr[j]; sb += S[j] * qr[j]; }
#pragma unroll
      for (int o = TPR / 2; o > 0; o >>= 1) {
        sa += __shfl_xor_sync(0xffffffffu, sa, o);
        sb += __shfl_xor_sync(0xffffffffu, sb, o);
      }
      const float u = (vv - dcy * sa) * m.y;
#pragma unroll
      for (int j = 0; j < KPT; ++j) S[j] = dcy * S[j] + u * kr[j];
      if (kpart == 0) o_raw[(size_t)(base + t) * hv * DV + h * DV + row0 + vrow] = dcy * sb + u * m.z;
    }
  }
  if (line > 0) {
    if constexpr (VEC == 4) {
#pragma unroll
      for (int g = 0; g < NG; ++g)
        *reinterpret_cast<float4*>(Sg + g * 4 * TPR + kpart * 4) = make_float4(S[4 * g], S[4 * g + 1], S[4 * g + 2], S[4 * g + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < KPT; ++j) Sg[kidx(j)] = S[j];
    }
  }
}

#define KERN_GDN_ENTRY(name, DK, DV, ROWS)                                                                             \
  extern "C" __global__ void __launch_bounds__(256)                                                                    \
      name(const __nv_bfloat16* qkv, const __nv_bfloat16* zba, float* o_raw, uint8_t* state, const int* lines,         \
           const int* cu_q, const float* A_log, const float* dt_bias, int seqs, int hk, int hv, int zba_stride,        \
           int b_off, int a_off, long long line_bytes, long long s_offset, int tb) {                                   \
    pdl_wait();                                                                                                        \
    gdn_body<DK, DV, ROWS>(qkv, zba, o_raw, state, lines, cu_q, A_log, dt_bias, seqs, hk, hv, zba_stride, b_off,       \
                           a_off, line_bytes, s_offset, tb < 1 ? 1 : (tb > GDN_TB ? GDN_TB : tb));                     \
  }

#define KERN_KDA_ENTRY(name, DK, DV, ROWS)                                                                             \
  extern "C" __global__ void __launch_bounds__(256)                                                                    \
      name(const __nv_bfloat16* qkv, const __nv_bfloat16* zba, float* o_raw, uint8_t* state, const int* lines,         \
           const int* cu_q, const float* A_log, const float* dt_bias, const __nv_bfloat16* gk, int seqs, int hk,       \
           int hv, int zba_stride, int b_off, int gk_stride, long long line_bytes, long long s_offset, int tb) {       \
    pdl_wait();                                                                                                        \
    gdn_body<DK, DV, ROWS, true>(qkv, zba, o_raw, state, lines, cu_q, A_log, dt_bias, seqs, hk, hv, zba_stride, b_off,  \
                                 0, line_bytes, s_offset, tb < 1 ? 1 : (tb > GDN_TB ? GDN_TB : tb), gk, gk_stride);    \
  }

// prefill chunks (ragged rows per sequence): grid [HV * DV / 16, seqs]
KERN_GDN_ENTRY(kern_gdn_rule_k128_v128, 128, 128, 16)
KERN_GDN_ENTRY(kern_gdn_rule_k64_v64, 64, 64, 16)
KERN_GDN_ENTRY(kern_gdn_rule_k32_v32, 32, 32, 16)
// decay per key channel (Kimi Delta Attention), ragged rows; dynamic shared memory (3 DK + ROWS + 4) * 4 bytes per staged token
KERN_KDA_ENTRY(kern_kda_rule_k128_v128, 128, 128, 16)
KERN_KDA_ENTRY(kern_kda_rule_k64_v64, 64, 64, 16)
// one row per sequence, unfused (the fused decode step is kern_gdn_step_*): grid [HV * DV / 16, seqs]
KERN_GDN_ENTRY(kern_gdn_rule_dec_k128_v128, 128, 128, 16)
KERN_GDN_ENTRY(kern_gdn_rule_dec_k64_v64, 64, 64, 16)
KERN_GDN_ENTRY(kern_gdn_rule_dec_k32_v32, 32, 32, 16)

// y = rmsnorm(o) * w * silu(z) per (token, value head): a warp per row of dv values (dv a multiple of 32, at most
// 256), grid [ceil(HV / 4), tokens], block 128.
extern "C" __global__ void __launch_bounds__(128)
    kern_gdn_gate_norm_bf16(const float* o_raw, const __nv_bfloat16* zba, __nv_bfloat16* out, const __nv_bfloat16* norm_w,
                            int tokens, int hv, int dv, int zba_stride, int z_off, float eps) {
  pdl_wait();
  const int t = blockIdx.y, h = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= tokens || h >= hv) return;
  const float* o = o_raw + ((size_t)t * hv + h) * dv;
  const __nv_bfloat16* z = zba + (size_t)t * zba_stride + z_off + h * dv;
  __nv_bfloat16* y = out + ((size_t)t * hv + h) * dv;
  if (dv == 128 && (zba_stride & 3) == 0 && (z_off & 3) == 0) {      // 16-byte loads of o, 8-byte loads of z and the weight
                                                                      // (rows of z must then start 8-byte aligned)
    const float4 v = *reinterpret_cast<const float4*>(o + lane * 4);
    const uint2 zu = *reinterpret_cast<const uint2*>(z + lane * 4);
    const uint2 wu = *reinterpret_cast<const uint2*>(norm_w + lane * 4);
    const float inv = rsqrtf(warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w) / 128.f + eps);
    const float2 z01 = unpack_bf16x2(zu.x), z23 = unpack_bf16x2(zu.y), w01 = unpack_bf16x2(wu.x), w23 = unpack_bf16x2(wu.y);
    *reinterpret_cast<uint2*>(y + lane * 4) =
        make_uint2(pack_bf16x2(v.x * inv * w01.x * silu(z01.x), v.y * inv * w01.y * silu(z01.y)),
                   pack_bf16x2(v.z * inv * w23.x * silu(z23.x), v.w * inv * w23.y * silu(z23.y)));
    return;
  }
  float ov[8], ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = i * 32 + lane;
    ov[i] = c < dv ? o[c] : 0.f;
    ss += ov[i] * ov[i];
  }
  const float inv = rsqrtf(warp_sum(ss) / (float)dv + eps);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = i * 32 + lane;
    if (c < dv) y[c] = __float2bfloat16(ov[i] * inv * __bfloat162float(norm_w[c]) * silu(__bfloat162float(z[c])));
  }
}

// ---- fused decode step -------------------------------------------------------------------------------------------
// One new token per sequence: a CTA owns one (sequence, value head) pair. The head's whole [DV, DK] f32 state comes in
// with bulk copies (one mbarrier; 64 KB in flight per CTA, three CTAs per SM) while the warps normalise q and k and
// fetch v and the gates; the rule then runs out of shared memory, the new state goes straight from registers to
// global memory, and the gated RMSNorm of the head's output closes the same launch. The step is bandwidth-bound: the
// roofline is two passes over the state at the copy bandwidth.
// Reference: tools/kernels-src/gdn_decode.cu:171 (kern_gdn_step_bf16: same fusion, one state tile per CTA).
// KDA = true: the decay is per key channel (Kimi Delta Attention): S[v, k] <- dec[k] S[v, k] before the delta update,
// dec[k] = exp(-exp(A_log[h]) softplus(gk[t, h, k] + dt_bias[h, k])); `gk` rows of HV * DK bf16 replace the scalar gate
// column `a` (dt_bias then holds HV * DK values).
template <int DK, int DV, bool KDA = false>
__device__ __forceinline__ void gdn_step_body(const __nv_bfloat16* qkv, const __nv_bfloat16* zba, __nv_bfloat16* out,
                                              uint8_t* state, const int* lines, const float* A_log, const float* dt_bias,
                                              const __nv_bfloat16* norm_w, int seqs, int hk, int hv, int zba_stride,
                                              int z_off, int b_off, int a_off, long long line_bytes, long long s_offset,
                                              float eps, const __nv_bfloat16* gk = nullptr, int gk_stride = 0) {
  constexpr int TPR = DK >= 64 ? 16 : DK / 4;   // lanes per value row; each holds DK / TPR keys in 16-byte groups
  constexpr int KPT = DK / TPR;
  constexpr int NG = KPT / 4;
  constexpr int RPP = 256 / TPR;                // value rows per pass
  constexpr int PASSES = DV / RPP;
  static_assert(KPT % 4 == 0 && DV % RPP == 0 && PASSES >= 1, "shape");
  constexpr uint32_t STATE_BYTES = DV * DK * 4;
  constexpr uint32_t PIECE = STATE_BYTES < 16384 ? STATE_BYTES : 16384;
  extern __shared__ __align__(128) float gdn_sm[];
  float* Ssm = gdn_sm;                          // [DV][DK]
  float* qs = Ssm + DV * DK;
  float* ks = qs + DK;
  float* vs = ks + DK;
  float* os = vs + DV;
  float* red = os + DV;                         // 8 partial sums + {decay, beta, k.q}
  uint64_t* bar = reinterpret_cast<uint64_t*>(red + 16);
  float* dec = reinterpret_cast<float*>(bar + 2);      // KDA: per-key decay [DK]
  const int h = blockIdx.x, s = blockIdx.y;
  if (s >= seqs) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int line = lines[s];
  if (line > 0 && !KERN_CHECK(state + (size_t)line * line_bytes, (size_t)line_bytes, SITE_STATE_SLOT)) line = 0;   // checked builds: a slot outside the pool is the null line
  uint8_t* Sg8 = state + (size_t)line * line_bytes + s_offset + (size_t)h * STATE_BYTES;
  if (tid == 0) {
    mbar_init(bar, 1);
    mbar_fence_init();
    if (line > 0) {
      mbar_expect_tx(bar, STATE_BYTES);
      for (uint32_t off = 0; off < STATE_BYTES; off += PIECE)
        bulk_load_1d(reinterpret_cast<uint8_t*>(Ssm) + off, Sg8 + off, PIECE, bar);
    }
  }
  const int kh = h / (hv / hk);
  const int conv_dim = 2 * hk * DK + hv * DV;
  const __nv_bfloat16* row = qkv + (size_t)s * conv_dim;
  if (warp == 0) {
    constexpr int QN = (DK + 31) / 32;
    float pq[QN], pk[QN];
    float q2 = 0.f, k2 = 0.f, qk = 0.f;
#pragma unroll
    for (int i = 0; i < QN; ++i) {
      const int c = i * 32 + lane;
      pq[i] = c < DK ? __bfloat162float(row[kh * DK + c]) : 0.f;
      pk[i] = c < DK ? __bfloat162float(row[hk * DK + kh * DK + c]) : 0.f;
      q2 += pq[i] * pq[i]; k2 += pk[i] * pk[i]; qk += pq[i] * pk[i];
    }
    q2 = warp_sum(q2); k2 = warp_sum(k2); qk = warp_sum(qk);
    const float qi = rsqrtf(q2 + 1e-6f) * rsqrtf((float)DK), ki = rsqrtf(k2 + 1e-6f);
#pragma unroll
    for (int i = 0; i < QN; ++i) {
      const int c = i * 32 + lane;
      if (c < DK) { qs[c] = pq[i] * qi; ks[c] = pk[i] * ki; }
    }
    if (lane == 0) red[10] = qk * qi * ki;
  } else if (warp == 1) {
    if (lane == 0) {
      const float av = __bfloat162float(zba[(size_t)s * zba_stride + a_off + h]) + dt_bias[h];
      const float sp = av > 20.f ? av : log1pf(__expf(av));
      const float bb = __bfloat162float(zba[(size_t)s * zba_stride + b_off + h]);
      red[8] = __expf(-__expf(A_log[h]) * sp);
      red[9] = __bfloat162float(__float2bfloat16(1.f / (1.f + __expf(-bb))));
    }
    if constexpr (KDA) {
      const float a_neg = -__expf(A_log[h]);
      for (int c = lane; c < DK; c += 32) {
        const float x = __bfloat162float(gk[(size_t)s * gk_stride + h * DK + c]) + dt_bias[h * DK + c];
        dec[c] = __expf(a_neg * (x > 20.f ? x : log1pf(__expf(x))));
      }
    }
  } else {
    for (int r = tid - 64; r < DV; r += 192) vs[r] = __bfloat162float(row[2 * hk * DK + h * DV + r]);
  }
  __syncthreads();                              // q, k, v, gates parked; the barrier's init is visible
  bool have = line > 0;
  if (have) {
    // every copy reads this GPU's own memory and completes; the limit only keeps a broken launch from spinning, and
    // a CTA that gave up reads the state with plain loads instead (same values), so no result depends on the limit
    bool ok = false;
    for (uint32_t i = 0; i < (1u << 22) && !ok; ++i) ok = mbar_try_wait(bar, 0) != 0;
    if (!__syncthreads_and(ok ? 1 : 0)) {
      const float4* src = reinterpret_cast<const float4*>(Sg8);
      for (int i = tid; i < (int)(STATE_BYTES / 16); i += 256) reinterpret_cast<float4*>(Ssm)[i] = src[i];
      __syncthreads();
    }
  }
  const float decay = KDA ? 1.f : red[8], beta = red[9], kq = red[10];
  const int vrow = tid / TPR, kpart = tid % TPR;
  float kr[KPT], qr[KPT], dr[KPT];
#pragma unroll
  for (int g = 0; g < NG; ++g) {
    const float4 k4 = *reinterpret_cast<const float4*>(ks + g * 4 * TPR + kpart * 4);
    const float4 q4 = *reinterpret_cast<const float4*>(qs + g * 4 * TPR + kpart * 4);
    kr[4 * g] = k4.x; kr[4 * g + 1] = k4.y; kr[4 * g + 2] = k4.z; kr[4 * g + 3] = k4.w;
    qr[4 * g] = q4.x; qr[4 * g + 1] = q4.y; qr[4 * g + 2] = q4.z; qr[4 * g + 3] = q4.w;
    if constexpr (KDA) {
      const float4 d4 = *reinterpret_cast<const float4*>(dec + g * 4 * TPR + kpart * 4);
      dr[4 * g] = d4.x; dr[4 * g + 1] = d4.y; dr[4 * g + 2] = d4.z; dr[4 * g + 3] = d4.w;
    } else {
      dr[4 * g] = dr[4 * g + 1] = dr[4 * g + 2] = dr[4 * g + 3] = red[8];
    }
  }
  (void)decay;
#pragma unroll
  for (int p = 0; p < PASSES; ++p) {
    const int r = p * RPP + vrow;
    float S[KPT];
#pragma unroll
    for (int g = 0; g < NG; ++g) {
      const float4 v = have ? *reinterpret_cast<const float4*>(Ssm + (size_t)r * DK + g * 4 * TPR + kpart * 4)
                            : make_float4(0.f, 0.f, 0.f, 0.f);
      S[4 * g] = v.x; S[4 * g + 1] = v.y; S[4 * g + 2] = v.z; S[4 * g + 3] = v.w;
    }
    // the decayed state first (a scalar per head, or a value per key channel), then both products on it
#pragma unroll
    for (int j = 0; j < KPT; ++j) S[j] *= dr[j];
    float sa = 0.f, sb = 0.f;
#pragma unroll
    for (int j = 0; j < KPT; ++j) { sa += S[j] * kr[j]; sb += S[j] * qr[j]; }
#pragma unroll
    for (int o = TPR / 2; o > 0; o >>= 1) {
      sa += __shfl_xor_sync(0xffffffffu, sa, o);
      sb += __shfl_xor_sync(0xffffffffu, sb, o);
    }
    const float u = (vs[r] - sa) * beta;
    if (have) {
      float* dst = reinterpret_cast<float*>(Sg8) + (size_t)r * DK;
#pragma unroll
      for (int g = 0; g < NG; ++g)
        *reinterpret_cast<float4*>(dst + g * 4 * TPR + kpart * 4) =
            make_float4(S[4 * g] + u * kr[4 * g], S[4 * g + 1] + u * kr[4 * g + 1], S[4 * g + 2] + u * kr[4 * g + 2],
                        S[4 * g + 3] + u * kr[4 * g + 3]);
    }
    if (kpart == 0) os[r] = sb + u * kq;
  }
  __syncthreads();
  // gated RMSNorm over the head's DV outputs
  float ss = 0.f;
  for (int i = tid; i < DV; i += 256) ss += os[i] * os[i];
  ss = warp_sum(ss);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) tot += red[w];
  const float inv = rsqrtf(tot / (float)DV + eps);
  for (int i = tid; i < DV; i += 256) {
    const float z = __bfloat162float(zba[(size_t)s * zba_stride + z_off + h * DV + i]);
    out[((size_t)s * hv + h) * DV + i] = __float2bfloat16(os[i] * inv * __bfloat162float(norm_w[i]) * silu(z));
  }
}

#define KERN_GDN_STEP_ENTRY(name, DK, DV)                                                                              \
  extern "C" __global__ void __launch_bounds__(256)                                                                    \
      name(const __nv_bfloat16* qkv, const __nv_bfloat16* zba, __nv_bfloat16* out, uint8_t* state, const int* lines,   \
           const float* A_log, const float* dt_bias, const __nv_bfloat16* norm_w, int seqs, int hk, int hv,            \
           int zba_stride, int z_off, int b_off, int a_off, long long line_bytes, long long s_offset, float eps) {     \
    pdl_wait();                                                                                                        \
    gdn_step_body<DK, DV>(qkv, zba, out, state, lines, A_log, dt_bias, norm_w, seqs, hk, hv, zba_stride, z_off, b_off,  \
                          a_off, line_bytes, s_offset, eps);                                                           \
  }

#define KERN_KDA_STEP_ENTRY(name, DK, DV)                                                                               \
  extern "C" __global__ void __launch_bounds__(256)                                                                    \
      name(const __nv_bfloat16* qkv, const __nv_bfloat16* zba, __nv_bfloat16* out, uint8_t* state, const int* lines,   \
           const float* A_log, const float* dt_bias, const __nv_bfloat16* norm_w, const __nv_bfloat16* gk, int seqs,   \
           int hk, int hv, int zba_stride, int z_off, int b_off, int gk_stride, long long line_bytes,                  \
           long long s_offset, float eps) {                                                                            \
    pdl_wait();                                                                                                        \
    gdn_step_body<DK, DV, true>(qkv, zba, out, state, lines, A_log, dt_bias, norm_w, seqs, hk, hv, zba_stride, z_off,   \
                                b_off, 0, line_bytes, s_offset, eps, gk, gk_stride);                                   \
  }

// grid [HV, seqs], block 256, dynamic shared memory DV * DK * 4 + (2 DK + 2 DV + 16) * 4 + 16 bytes (+ DK * 4 for KDA)
KERN_GDN_STEP_ENTRY(kern_gdn_step_k128_v128, 128, 128)
KERN_GDN_STEP_ENTRY(kern_gdn_step_k64_v64, 64, 64)
KERN_GDN_STEP_ENTRY(kern_gdn_step_k32_v32, 32, 32)
// per-key decay (Kimi Delta Attention) decode step: `gk` [tokens, HV * DK] bf16 gate rows, dt_bias [HV * DK]
KERN_KDA_STEP_ENTRY(kern_kda_step_k128_v128, 128, 128)
KERN_KDA_STEP_ENTRY(kern_kda_step_k64_v64, 64, 64)
