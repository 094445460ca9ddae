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
// reference takes chunked prefill as a mined kernel. Here one kernel body serves both: the state tile
// lives in shared memory for the whole chunk of a sequence, tokens are walked in order.
#include "common.cuh"

using namespace kern;

// ---- causal conv (width <= 4) + SiLU ----------------------------------------------------------------
// x: [tokens][x_stride] (the q|k|v channels are the first conv_dim of a row), y: [tokens][conv_dim]
// w: [conv_dim][width] bf16, bias optional. cu_q: [seqs+1] row starts (nullptr: one row per sequence).
// grid [seqs, ceil(conv_dim / 256)], block 256: a thread owns one channel and walks its sequence's rows.
extern "C" __global__ void __launch_bounds__(256)
    kern_gdn_conv_bf16(const __nv_bfloat16* x, __nv_bfloat16* y, uint8_t* state, const int* lines, const int* cu_q,
                       const __nv_bfloat16* w, const __nv_bfloat16* bias, int seqs, int conv_dim, int width, int x_stride,
                       long long line_bytes) {
  pdl_wait();
  const int s = blockIdx.x;
  const int c = blockIdx.y * 256 + threadIdx.x;
  if (s >= seqs || c >= conv_dim) return;
  const int line = lines[s];
  const int r0 = cu_q ? cu_q[s] : s, r1 = cu_q ? cu_q[s + 1] : s + 1;
  if (r1 <= r0) return;
  __nv_bfloat16* win = reinterpret_cast<__nv_bfloat16*>(state + (size_t)line * line_bytes);   // [(width-1)][conv_dim]
  float hist[3] = {0.f, 0.f, 0.f};
  for (int j = 0; j < width - 1; ++j) hist[j] = line > 0 ? __bfloat162float(win[(size_t)j * conv_dim + c]) : 0.f;
  float wt[4] = {0.f, 0.f, 0.f, 0.f};
  for (int j = 0; j < width; ++j) wt[j] = __bfloat162float(w[(size_t)c * width + j]);
  const float bs = bias ? __bfloat162float(bias[c]) : 0.f;
  for (int r = r0; r < r1; ++r) {
    const float cur = __bfloat162float(x[(size_t)r * x_stride + c]);
    float acc = bs + wt[width - 1] * cur;
    for (int j = 0; j < width - 1; ++j) acc += wt[j] * hist[j];
    y[(size_t)r * conv_dim + c] = __float2bfloat16(silu(acc));
    for (int j = 0; j + 1 < width - 1; ++j) hist[j] = hist[j + 1];
    if (width > 1) hist[width - 2] = cur;
  }
  if (line > 0)
    for (int j = 0; j < width - 1; ++j) win[(size_t)j * conv_dim + c] = __float2bfloat16(hist[j]);
}

// ---- gated delta rule ---------------------------------------------------------------------------------
// qkv: conv output [tokens][conv_dim] laid out [q: HK*DK | k: HK*DK | v: HV*DV]
// zba: [tokens][zba_stride] with z at z_off (HV*DV), b at b_off (HV), a at a_off (HV)   (bf16)
// out: [tokens][HV*DV] bf16.  A_log, dt_bias: f32 [HV].  norm_w: bf16 [DV].
// grid [HV, seqs], block 256, dyn smem = (DV * (DK + 256 / DV) + 2 * DK + DV) * 4 bytes.
// 256 / DV threads share a value row, each taking every (256 / DV)-th key column.
template <int DK, int DV>
__device__ __forceinline__ void gdn_body(const __nv_bfloat16* qkv, const __nv_bfloat16* zba, __nv_bfloat16* out, uint8_t* state,
                                         const int* lines, const int* cu_q, const float* A_log, const float* dt_bias,
                                         const __nv_bfloat16* norm_w, int seqs, int hk, int hv, int zba_stride, int z_off,
                                         int b_off, int a_off, long long line_bytes, long long s_offset, float eps) {
  extern __shared__ float sm[];
  constexpr int TPR = 256 / DV;       // threads per value row
  constexpr int KPT = DK / TPR;       // k elements per thread (interleaved: k = j * TPR + part)
  constexpr int LD = DK + TPR;        // row stride = TPR mod 32 banks: a warp's 32 (row, part) pairs hit 32 banks
  float* S = sm;                      // [DV][LD]
  float* qs = S + DV * LD;            // [DK]
  float* ks = qs + DK;               // [DK]
  float* os = ks + DK;               // [DV] output before the norm
  __shared__ float red[32];
  const int h = blockIdx.x, s = blockIdx.y;
  if (s >= seqs) return;
  const int line = lines[s];
  const int r0 = cu_q ? cu_q[s] : s, r1 = cu_q ? cu_q[s + 1] : s + 1;
  if (r1 <= r0) return;
  const int kh = h / (hv / hk);
  const int conv_dim = 2 * hk * DK + hv * DV;
  float* Sg = reinterpret_cast<float*>(state + (size_t)line * line_bytes + s_offset) + (size_t)h * DV * DK;
  const int tid = threadIdx.x;
  for (int i = tid; i < DV * DK; i += 256) S[(i / DK) * LD + (i % DK)] = line > 0 ? Sg[i] : 0.f;
  const int vrow = tid / TPR, kpart = tid % TPR;
  const float a_neg = -__expf(A_log[h]);
  const float dtb = dt_bias[h];
  const int warp = tid >> 5, lane = tid & 31;
  __syncthreads();
  for (int r = r0; r < r1; ++r) {
    const __nv_bfloat16* row = qkv + (size_t)r * conv_dim;
    // q, k with l2 norm (all threads cooperate: DK <= 256)
    float qv = 0.f, kv = 0.f;
    if (tid < DK) {
      qv = __bfloat162float(row[kh * DK + tid]);
      kv = __bfloat162float(row[hk * DK + kh * DK + tid]);
    }
    float q2 = warp_sum(qv * qv), k2 = warp_sum(kv * kv);
    if (lane == 0) { red[warp] = q2; red[8 + warp] = k2; }
    __syncthreads();
    float qn = 0.f, kn = 0.f;
    for (int i = 0; i < 8; ++i) { qn += red[i]; kn += red[8 + i]; }
    if (tid < DK) {
      qs[tid] = qv * rsqrtf(qn + 1e-6f) * rsqrtf((float)DK);
      ks[tid] = kv * rsqrtf(kn + 1e-6f);
    }
    const float av = __bfloat162float(zba[(size_t)r * zba_stride + a_off + h]) + dtb;
    const float sp = av > 20.f ? av : log1pf(__expf(av));
    const float decay = __expf(a_neg * sp);
    const float bb = __bfloat162float(zba[(size_t)r * zba_stride + b_off + h]);
    const float beta = __bfloat162float(__float2bfloat16(1.f / (1.f + __expf(-bb))));
    const float vv = __bfloat162float(row[2 * hk * DK + h * DV + vrow]);
    __syncthreads();
    // S *= decay; sk = S k (this thread's part of its row)
    float* Srow = S + vrow * LD + kpart;
    float sk = 0.f;
#pragma unroll 8
    for (int j = 0; j < KPT; ++j) {
      const float sv = Srow[j * TPR] * decay;
      Srow[j * TPR] = sv;
      sk += sv * ks[j * TPR + kpart];
    }
#pragma unroll
    for (int o = TPR / 2; o > 0; o >>= 1) sk += __shfl_xor_sync(0xffffffffu, sk, o);
    const float u = (vv - sk) * beta;
    float oq = 0.f;
#pragma unroll 8
    for (int j = 0; j < KPT; ++j) {
      const float sv = Srow[j * TPR] + u * ks[j * TPR + kpart];
      Srow[j * TPR] = sv;
      oq += sv * qs[j * TPR + kpart];
    }
#pragma unroll
    for (int o = TPR / 2; o > 0; o >>= 1) oq += __shfl_xor_sync(0xffffffffu, oq, o);
    if (kpart == 0) os[vrow] = oq;
    __syncthreads();
    // gated RMSNorm over DV: y = o * rsqrt(mean(o^2) + eps) * w * silu(z)
    float ov = tid < DV ? os[tid] : 0.f;
    float o2 = warp_sum(ov * ov);
    if (lane == 0) red[16 + warp] = o2;
    __syncthreads();
    float on = 0.f;
    for (int i = 0; i < 8; ++i) on += red[16 + i];
    if (tid < DV) {
      const float z = __bfloat162float(zba[(size_t)r * zba_stride + z_off + h * DV + tid]);
      const float y = ov * rsqrtf(on / (float)DV + eps) * __bfloat162float(norm_w[tid]) * silu(z);
      out[(size_t)r * hv * DV + h * DV + tid] = __float2bfloat16(y);
    }
    __syncthreads();
  }
  if (line > 0)
    for (int i = tid; i < DV * DK; i += 256) Sg[i] = S[(i / DK) * LD + (i % DK)];
}

#define KERN_GDN_ENTRY(name, DK, DV)                                                                                  \
  extern "C" __global__ void __launch_bounds__(256)                                                                   \
      name(const __nv_bfloat16* qkv, const __nv_bfloat16* zba, __nv_bfloat16* out, uint8_t* state, const int* lines,  \
           const int* cu_q, const float* A_log, const float* dt_bias, const __nv_bfloat16* norm_w, int seqs, int hk,  \
           int hv, int zba_stride, int z_off, int b_off, int a_off, long long line_bytes, long long s_offset,         \
           float eps) {                                                                                               \
    pdl_wait();                                                                                                       \
    gdn_body<DK, DV>(qkv, zba, out, state, lines, cu_q, A_log, dt_bias, norm_w, seqs, hk, hv, zba_stride, z_off,       \
                     b_off, a_off, line_bytes, s_offset, eps);                                                        \
  }

KERN_GDN_ENTRY(kern_gdn_rule_k128_v128, 128, 128)
KERN_GDN_ENTRY(kern_gdn_rule_k64_v64, 64, 64)
KERN_GDN_ENTRY(kern_gdn_rule_k32_v32, 32, 32)
