// Mixers that carry a state of fixed size per request instead of keys and values per position:
//
//   * a short causal convolution over time per channel, followed by SiLU, whose last taps-1 inputs are state;
//   * the gated delta rule: per head a matrix S [key channels, value channels] with a decay per key channel,
//       S <- diag(g_t) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t;
//   * the stabilised matrix memory (mLSTM): per head S, a normaliser n and a running maximum m of the log gates,
//       m_t = max(f_t + m_{t-1}, i_t);  a = exp(f_t + m_{t-1} - m_t);  b = exp(i_t - m_t);
//       S <- a S + b k_t v_t^T;  n <- a n + b k_t;  o_t = S^T q_t / (max(|n . q_t|, exp(-m_t)) + 1e-6);
//   * the RMS norm per head with a weight and a sigmoid gate that follows both.
//
// A step is a batch of requests, each bringing a run of consecutive tokens (cu_q[r] .. cu_q[r+1]) that continues
// from the request's state slot (state_slots[r]).  Everything that enters a recurrence is float32: the inputs are
// the float32 outputs of the projections, gates and decays are computed here, the state lives in float32.  The
// scan kernels give one CTA a (request, head): SPLIT neighbouring lanes share one value channel, i.e. one column
// of S, each holding a contiguous part of its key channels in registers, so a token costs each thread DK / SPLIT
// steps and two small shuffle reductions (the column's dot products with k and with q, added in a fixed tree);
// the per-token vectors (q, k, decays, gates) of a chunk of tokens are staged and prepared in shared memory by
// the whole CTA.  A token's result
// depends on the state and the tokens before it only, in an order of operations that is the same however the
// sequence was cut into steps.
#include "common.cuh"

namespace {

constexpr int MAX_TAPS = 16;

__device__ __forceinline__ float rc_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float rc_softplus(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ void rc_store(void* out, int dtype, size_t i, float v) {
  if (dtype == CO_BF16) ((__nv_bfloat16*)out)[i] = __float2bfloat16_rn(v);
  else ((float*)out)[i] = v;
}

// ---------------------------------------------------------------------------------
// y[t, c] = silu(sum_j taps[c, j] * x[t - (n-1) + j, c]); inputs before the step's first token of a request come
// from its state [n-1, C] (oldest first), which holds zeros for a request that has just been admitted.
// ---------------------------------------------------------------------------------
__global__ void short_conv_silu_kernel(const float* __restrict__ x, long ldx, float* __restrict__ y, long ldy,
                                       const void* __restrict__ taps, int taps_dtype, int n, int C,
                                       const float* __restrict__ state, long state_stride,
                                       const int* __restrict__ token_req, const int* __restrict__ cu_q,
                                       const int* __restrict__ state_slots, int T) {
  co_pdl_launch_dependents();
  co_pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)T * C) return;
  const int t = (int)(idx / C), c = (int)(idx % C);
  const int r = token_req[t];
  const int start = cu_q[r];
  const int i = t - start;
  const float* st = state + (size_t)state_slots[r] * state_stride;
  float acc = 0.f;
  for (int j = 0; j < n; ++j) {
    const int p = i - (n - 1) + j;
    const float xv = p >= 0 ? x[(size_t)(start + p) * ldx + c] : st[(size_t)(n - 1 + p) * C + c];
    acc = fmaf(co_load_any(taps, taps_dtype, (size_t)c * n + j), xv, acc);
  }
  y[(size_t)t * ldy + c] = acc / (1.0f + expf(-acc));
}

// The state after the step: the last n-1 inputs of each request, taken from the step's rows and, where the
// step brought fewer than n-1 tokens, from the old state.
__global__ void short_conv_state_kernel(const float* __restrict__ x, long ldx, int n, int C, float* __restrict__ state,
                                        long state_stride, const int* __restrict__ cu_q,
                                        const int* __restrict__ state_slots, int B) {
  co_pdl_launch_dependents();
  co_pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)B * C) return;
  const int r = (int)(idx / C), c = (int)(idx % C);
  const int start = cu_q[r], len = cu_q[r + 1] - start;
  if (len <= 0) return;
  float* st = state + (size_t)state_slots[r] * state_stride;
  float keep[MAX_TAPS];
  for (int s = 0; s < n - 1; ++s) {
    const int p = len - (n - 1) + s;
    keep[s] = p >= 0 ? x[(size_t)(start + p) * ldx + c] : st[(size_t)(n - 1 + p) * C + c];
  }
  for (int s = 0; s < n - 1; ++s) st[(size_t)s * C + c] = keep[s];
}

// ---------------------------------------------------------------------------------
// What both scans share: the output of a chunk of tokens (os [CT][dvp], one head) is divided by its root mean
// square over the value channels, multiplied by a weight and by the sigmoid of a gate's pre-activation, and
// written in the output's dtype.  A warp takes a token.
// ---------------------------------------------------------------------------------
struct HeadOut {
  void* out; int out_dtype; long ldo;          // [T, heads * dv]
  const void* weight; int weight_dtype;        // [dv] shared by the heads (weight_stride 0) or [heads * dv]
  int weight_stride;
  const float* gate; long ldg;                 // pre-activations [T, heads * dv]
  float eps, out_scale;
  // When the columns of a head are split over several CTAs (a long prompt of few requests: more SMs at work), no CTA sees a
  // whole head: the scans then leave the unnormalised outputs in `raw` [T, heads * dv] and a second kernel applies norm,
  // weight and gate, in the same order of operations.  `nm_next`: where the matrix memory's n and m of each (request,
  // head) wait until every CTA of the head has read the old ones ([B][heads][dk + 1]).
  float* raw; long ldr;
  float* nm_next;
  int gate_act;                                // what the gate's pre-activation passes: 0 sigmoid, 1 SiLU
};

__device__ __forceinline__ void head_out_chunk(const HeadOut& E, const float* os, int dvp, int dv, int nt, int row0, int h) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  for (int i = warp; i < nt; i += warps) {
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) ss = fmaf(os[i * dvp + c], os[i * dvp + c], ss);
    ss = co_warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)dv + E.eps);
    const size_t row = (size_t)(row0 + i);
#pragma unroll 4
    for (int c = lane; c < dv; c += 32) {
      const float w = co_load_any(E.weight, E.weight_dtype, (size_t)h * E.weight_stride + c);
      const float z = E.gate[row * E.ldg + (size_t)h * dv + c];
      const float g = E.gate_act == 1 ? z * rc_sigmoid(z) : rc_sigmoid(z);
      rc_store(E.out, E.out_dtype, row * E.ldo + (size_t)h * dv + c, os[i * dvp + c] * inv * w * g * E.out_scale);
    }
  }
}

// The unnormalised outputs of a chunk for the CTA's columns (see HeadOut::raw).
__device__ __forceinline__ void raw_out_chunk(const HeadOut& E, const float* os, int dvp, int dv, int colbase, int nt, int row0, int h) {
  for (int e = threadIdx.x; e < nt * dvp; e += blockDim.x) {
    const int i = e / dvp, c = e % dvp;
    if (colbase + c < dv) E.raw[(size_t)(row0 + i) * E.ldr + (size_t)h * dv + colbase + c] = os[e];
  }
}

// Norm, weight and gate of whole heads from the unnormalised outputs: 16 tokens of a head per CTA, through the same
// function and therefore the same order of operations as the scans' own epilogue.
__global__ void __launch_bounds__(256) head_norm_gate_kernel(HeadOut E, int T, int dv) {
  extern __shared__ __align__(16) float smem[];
  co_pdl_launch_dependents();
  co_pdl_wait();
  const int row0 = blockIdx.x * 16, h = blockIdx.y, nt = min(16, T - row0);
  for (int e = threadIdx.x; e < nt * dv; e += blockDim.x) {
    const int i = e / dv, c = e % dv;
    smem[e] = E.raw[(size_t)(row0 + i) * E.ldr + (size_t)h * dv + c];
  }
  __syncthreads();
  head_out_chunk(E, smem, dv, dv, nt, row0, h);
}

// n and m of the matrix memory from the side into the state (see HeadOut::nm_next).
__global__ void memory_nm_commit_kernel(const float* __restrict__ nm, float* __restrict__ state, long state_stride,
                                        const int* __restrict__ state_slots, const int* __restrict__ cu_q, int heads, int dk, int dv) {
  co_pdl_launch_dependents();
  co_pdl_wait();
  const int r = blockIdx.x, h = blockIdx.y;
  if (cu_q[r + 1] - cu_q[r] <= 0) return;
  float* slot = state + (size_t)state_slots[r] * state_stride;
  const float* from = nm + ((size_t)r * heads + h) * (dk + 1);
  for (int d = threadIdx.x; d < dk; d += blockDim.x) slot[(size_t)heads * dk * dv + (size_t)h * dk + d] = from[d];
  if (threadIdx.x == 0) slot[(size_t)heads * dk * dv + (size_t)heads * dk + h] = from[dk];
}

// ---------------------------------------------------------------------------------
// How a scan's CTA is laid out.  SPLIT neighbouring lanes share CP neighbouring columns of S; each holds DP = DK / SPLIT
// contiguous key channels of them in registers (CP * DP values).  A token then costs a thread 3 DP / 4 vector loads
// from shared memory for 4 CP DP multiply-adds, and 2 CP shuffle reductions over SPLIT lanes, added in a fixed tree.
// The per-token vectors lie in shared memory with each lane's part padded apart so that the SPLIT parts fall on
// different banks.
// ---------------------------------------------------------------------------------
template <int DK, int SPLIT>
struct ScanShape {
  static constexpr int DP = DK / SPLIT;
  static constexpr int STRIDE = DP + (((DP / 4) % 2 == 0) ? 4 : 0);   // an odd number of 16-byte units
  static constexpr int ROW = SPLIT * STRIDE;
  static_assert(DK % SPLIT == 0 && DP % 4 == 0, "a lane's part is a whole number of 16-byte units");
  __device__ static __forceinline__ int at(int d) { return (d / DP) * STRIDE + d % DP; }
};

// A thread's part of S (CP columns by DP key channels) from and to the state [dk][dv]: 16-byte vectors over the
// columns where four of them are whole and aligned, single values otherwise.
template <int CP, int DP>
__device__ __forceinline__ void scan_state_load(float (&S)[CP][DP], const float* __restrict__ st, int d0, int col0, int dk, int dv) {
  if (CP % 4 == 0 && (dv & 3) == 0 && col0 + CP <= dv && (((uintptr_t)st) & 15) == 0) {
#pragma unroll
    for (int d = 0; d < DP; ++d)
#pragma unroll
      for (int c = 0; c + 3 < CP; c += 4) {
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (d0 + d < dk) x = *reinterpret_cast<const float4*>(st + (size_t)(d0 + d) * dv + col0 + c);
        S[c][d] = x.x; S[c + 1][d] = x.y; S[c + 2][d] = x.z; S[c + 3][d] = x.w;
      }
    return;
  }
#pragma unroll
  for (int c = 0; c < CP; ++c)
#pragma unroll
    for (int d = 0; d < DP; ++d) S[c][d] = (d0 + d < dk && col0 + c < dv) ? st[(size_t)(d0 + d) * dv + col0 + c] : 0.f;
}
template <int CP, int DP>
__device__ __forceinline__ void scan_state_store(const float (&S)[CP][DP], float* __restrict__ st, int d0, int col0, int dk, int dv) {
  if (CP % 4 == 0 && (dv & 3) == 0 && col0 + CP <= dv && (((uintptr_t)st) & 15) == 0) {
#pragma unroll
    for (int d = 0; d < DP; ++d)
#pragma unroll
      for (int c = 0; c + 3 < CP; c += 4)
        if (d0 + d < dk)
          *reinterpret_cast<float4*>(st + (size_t)(d0 + d) * dv + col0 + c) = make_float4(S[c][d], S[c + 1][d], S[c + 2][d], S[c + 3][d]);
    return;
  }
#pragma unroll
  for (int c = 0; c < CP; ++c)
#pragma unroll
    for (int d = 0; d < DP; ++d)
      if (d0 + d < dk && col0 + c < dv) st[(size_t)(d0 + d) * dv + col0 + c] = S[c][d];
}

template <int DP>
__device__ __forceinline__ void scan_fetch(float4 (&r)[DP / 4], const float* from) {
#pragma unroll
  for (int d = 0; d < DP / 4; ++d) r[d] = reinterpret_cast<const float4*>(from)[d];
}

template <int SPLIT>
__device__ __forceinline__ float split_sum(float v) {
#pragma unroll
  for (int o = SPLIT / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---------------------------------------------------------------------------------
// Gated delta rule.
// ---------------------------------------------------------------------------------
struct DeltaIn {
  const float* q; const float* k; const float* v; long ld_qkv;   // after convolution and SiLU: [T, kv_heads*dk], .., [T, heads*dv]
  const float* beta; long ld_beta;                               // pre-activation of beta [T, heads]
  const float* step; long ld_step;                               // pre-activation of the step size [T, heads*dc] (bias not added)
  const void* step_bias; int step_bias_dtype;                    // [heads*dc]; dc = decay_channels
  const void* rate_log; int rate_log_dtype;                      // [heads]: decay = exp(-exp(rate_log) * softplus(step + bias))
  float* state; long state_stride;                               // per slot: S [heads, dk, dv]
  const int* cu_q; const int* state_slots;
  int heads, kv_heads, dk, dv;
  int decay_channels;                                            // dk: a decay per head and key channel; 1: one per head
};

// The tokens of a staged chunk, one after the other, for the thread's part of S (see ScanShape).
template <typename L, int CP, int SPLIT>
__device__ __forceinline__ void delta_tokens(float (&S)[CP][L::DP], const float* qs, const float* ks, const float* gs, const float* vs,
                                             const float* betas, float* os, int nt, int part, int col0, int dvp) {
  constexpr int DP = L::DP, ROW = L::ROW;
  // The vectors of token i + 1 are fetched into registers before token i is worked on: the stores of a token's
  // outputs would otherwise hold the next token's loads back.
  float4 kc[DP / 4], gc[DP / 4], qc[DP / 4];
  scan_fetch<DP>(kc, ks + part * L::STRIDE);
  scan_fetch<DP>(gc, gs + part * L::STRIDE);
  scan_fetch<DP>(qc, qs + part * L::STRIDE);
  for (int i = 0; i < nt; ++i) {
    float4 kn[DP / 4], gn[DP / 4], qn[DP / 4];
    const int nx = min(i + 1, nt - 1) * ROW + part * L::STRIDE;
    scan_fetch<DP>(kn, ks + nx); scan_fetch<DP>(gn, gs + nx); scan_fetch<DP>(qn, qs + nx);
    float dot[CP][2];
#pragma unroll
    for (int c = 0; c < CP; ++c) dot[c][0] = dot[c][1] = 0.f;
#pragma unroll
    for (int d = 0; d < DP / 4; ++d) {
      const float4 gg = gc[d], kk = kc[d];
#pragma unroll
      for (int c = 0; c < CP; ++c) {
        S[c][4 * d] *= gg.x; S[c][4 * d + 1] *= gg.y; S[c][4 * d + 2] *= gg.z; S[c][4 * d + 3] *= gg.w;
        dot[c][0] = fmaf(S[c][4 * d], kk.x, dot[c][0]); dot[c][1] = fmaf(S[c][4 * d + 1], kk.y, dot[c][1]);
        dot[c][0] = fmaf(S[c][4 * d + 2], kk.z, dot[c][0]); dot[c][1] = fmaf(S[c][4 * d + 3], kk.w, dot[c][1]);
      }
    }
    float u[CP];
#pragma unroll
    for (int c = 0; c < CP; ++c) u[c] = betas[i] * (vs[i * dvp + col0 + c] - split_sum<SPLIT>(dot[c][0] + dot[c][1]));
#pragma unroll
    for (int c = 0; c < CP; ++c) dot[c][0] = dot[c][1] = 0.f;
#pragma unroll
    for (int d = 0; d < DP / 4; ++d) {
      const float4 kk = kc[d], qq = qc[d];
#pragma unroll
      for (int c = 0; c < CP; ++c) {
        S[c][4 * d] = fmaf(kk.x, u[c], S[c][4 * d]); S[c][4 * d + 1] = fmaf(kk.y, u[c], S[c][4 * d + 1]);
        S[c][4 * d + 2] = fmaf(kk.z, u[c], S[c][4 * d + 2]); S[c][4 * d + 3] = fmaf(kk.w, u[c], S[c][4 * d + 3]);
        dot[c][0] = fmaf(S[c][4 * d], qq.x, dot[c][0]); dot[c][1] = fmaf(S[c][4 * d + 1], qq.y, dot[c][1]);
        dot[c][0] = fmaf(S[c][4 * d + 2], qq.z, dot[c][0]); dot[c][1] = fmaf(S[c][4 * d + 3], qq.w, dot[c][1]);
      }
    }
#pragma unroll
    for (int c = 0; c < CP; ++c) {
      const float o = split_sum<SPLIT>(dot[c][0] + dot[c][1]);
      if (part == 0) os[i * dvp + col0 + c] = o;
    }
#pragma unroll
    for (int d = 0; d < DP / 4; ++d) { kc[d] = kn[d]; gc[d] = gn[d]; qc[d] = qn[d]; }
  }
}

template <int DK, int CT, int SPLIT, int CP>
__global__ void __launch_bounds__(512) gated_delta_scan_kernel(DeltaIn P, HeadOut E) {
  using L = ScanShape<DK, SPLIT>;
  constexpr int DP = L::DP, ROW = L::ROW;
  extern __shared__ __align__(16) float smem[];
  co_pdl_launch_dependents();
  co_pdl_wait();
  const int r = blockIdx.x, h = blockIdx.y;
  const int part = threadIdx.x % SPLIT, col0 = (threadIdx.x / SPLIT) * CP, d0 = part * DP;
  const int dk = P.dk, dv = P.dv, dvp = (blockDim.x / SPLIT) * CP;
  const int colbase = blockIdx.z * dvp;        // this CTA's first column of the head
  const int start = P.cu_q[r], len = P.cu_q[r + 1] - start;
  if (len <= 0) return;
  const int g = h / (P.heads / P.kv_heads);
  float* qs = smem;                    // [CT][ROW]
  float* ks = qs + CT * ROW;           // [CT][ROW]
  float* gs = ks + CT * ROW;           // [CT][ROW]
  float* vs = gs + CT * ROW;           // [CT][dvp]
  float* os = vs + CT * dvp;           // [CT][dvp]
  float* betas = os + CT * dvp;        // [CT]
  float* S_state = P.state + (size_t)P.state_slots[r] * P.state_stride + (size_t)h * dk * dv;
  float S[CP][DP];
  scan_state_load<CP, DP>(S, S_state, d0, colbase + col0, dk, dv);
  const float rate = expf(co_load_any(P.rate_log, P.rate_log_dtype, h));
  const float q_scale = 1.0f / sqrtf((float)dk);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;

  for (int c0 = 0; c0 < len; c0 += CT) {
    const int nt = min(CT, len - c0), row0 = start + c0;
#pragma unroll 8
    for (int e = threadIdx.x; e < nt * DK; e += blockDim.x) {      // unrolled: the loads of a thread are in flight together
      const int i = e / DK, d = e % DK;
      const size_t row = (size_t)(row0 + i);
      float qv = 0.f, kv = 0.f, gv = 1.f;
      if (d < dk) {
        qv = P.q[row * P.ld_qkv + (size_t)g * dk + d];
        kv = P.k[row * P.ld_qkv + (size_t)g * dk + d];
        const size_t sc = P.decay_channels == 1 ? (size_t)h : (size_t)h * dk + d;
        const float z = P.step[row * P.ld_step + sc] + co_load_any(P.step_bias, P.step_bias_dtype, sc);
        gv = expf(-rate * rc_softplus(z));
      }
      const int o = i * ROW + L::at(d);
      qs[o] = qv; ks[o] = kv; gs[o] = gv;
    }
#pragma unroll 8
    for (int e = threadIdx.x; e < nt * dvp; e += blockDim.x) {
      const int i = e / dvp, c = e % dvp;
      vs[e] = colbase + c < dv ? P.v[(size_t)(row0 + i) * P.ld_qkv + (size_t)h * dv + colbase + c] : 0.f;
    }
    if (threadIdx.x < nt) betas[threadIdx.x] = rc_sigmoid(P.beta[(size_t)(row0 + threadIdx.x) * P.ld_beta + h]);
    __syncthreads();
    // q and k become unit vectors (q also divided by sqrt(dk)): a warp per token
    for (int i = warp; i < nt; i += warps) {
      float sq = 0.f, sk = 0.f;
      for (int d = lane; d < DK; d += 32) {
        const float a = qs[i * ROW + L::at(d)], b = ks[i * ROW + L::at(d)];
        sq = fmaf(a, a, sq); sk = fmaf(b, b, sk);
      }
      sq = co_warp_sum(sq); sk = co_warp_sum(sk);
      const float iq = q_scale / sqrtf(sq + 1e-6f), ik = 1.0f / sqrtf(sk + 1e-6f);
      for (int d = lane; d < DK; d += 32) { qs[i * ROW + L::at(d)] *= iq; ks[i * ROW + L::at(d)] *= ik; }
    }
    __syncthreads();
    delta_tokens<L, CP, SPLIT>(S, qs, ks, gs, vs, betas, os, nt, part, col0, dvp);
    __syncthreads();
    if (E.raw) raw_out_chunk(E, os, dvp, dv, colbase, nt, row0, h);
    else head_out_chunk(E, os, dvp, dv, nt, row0, h);
    __syncthreads();
  }
  scan_state_store<CP, DP>(S, S_state, d0, colbase + col0, dk, dv);
}

// ---------------------------------------------------------------------------------
// The same scan for long prompts: what the plain kernel computes while it stages a chunk (unit-norm q and k, decays, beta)
// is made ONCE per token by delta_prepare_kernel, parallel over the tokens, so that this kernel stages by asynchronous
// copies, two chunks deep, and the CTAs that share a head (64 value channels each) repeat nothing but copies.
// prep: [T][kv_heads*dk (q) | kv_heads*dk (k) | heads*dk (decay) | heads (beta)].
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async4(float* smem_dst, const float* src) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(a), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit_group() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__global__ void __launch_bounds__(128) delta_prepare_kernel(DeltaIn P, float* __restrict__ prep, long ld_prep) {
  co_pdl_launch_dependents();
  co_pdl_wait();
  const size_t t = blockIdx.x;
  const int dk = P.dk, G = P.kv_heads, H = P.heads;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  float* out = prep + t * ld_prep;
  const float q_scale = 1.0f / sqrtf((float)dk);
  for (int g = warp; g < G; g += warps) {          // the same sums, in the same order, as the plain kernel's staging
    const float* q = P.q + t * P.ld_qkv + (size_t)g * dk;
    const float* k = P.k + t * P.ld_qkv + (size_t)g * dk;
    float sq = 0.f, sk = 0.f;
    for (int d = lane; d < dk; d += 32) { sq = fmaf(q[d], q[d], sq); sk = fmaf(k[d], k[d], sk); }
    sq = co_warp_sum(sq); sk = co_warp_sum(sk);
    const float iq = q_scale / sqrtf(sq + 1e-6f), ik = 1.0f / sqrtf(sk + 1e-6f);
    for (int d = lane; d < dk; d += 32) { out[(size_t)g * dk + d] = q[d] * iq; out[(size_t)(G + g) * dk + d] = k[d] * ik; }
  }
  for (int e = threadIdx.x; e < H * dk; e += blockDim.x) {
    const float rate = expf(co_load_any(P.rate_log, P.rate_log_dtype, e / dk));
    const size_t sc = P.decay_channels == 1 ? (size_t)(e / dk) : (size_t)e;
    const float z = P.step[t * P.ld_step + sc] + co_load_any(P.step_bias, P.step_bias_dtype, sc);
    out[(size_t)2 * G * dk + e] = expf(-rate * rc_softplus(z));
  }
  for (int e = threadIdx.x; e < H; e += blockDim.x) out[(size_t)(2 * G + H) * dk + e] = rc_sigmoid(P.beta[t * P.ld_beta + e]);
}

template <int DK, int CT, int SPLIT, int CP>
__global__ void __launch_bounds__(512) gated_delta_scan_pre_kernel(DeltaIn P, HeadOut E, const float* __restrict__ prep, long ld_prep) {
  using L = ScanShape<DK, SPLIT>;
  constexpr int DP = L::DP, ROW = L::ROW;
  extern __shared__ __align__(16) float smem[];
  co_pdl_launch_dependents();
  co_pdl_wait();
  const int r = blockIdx.x, h = blockIdx.y;
  const int part = threadIdx.x % SPLIT, col0 = (threadIdx.x / SPLIT) * CP, d0 = part * DP;
  const int dk = P.dk, dv = P.dv, dvp = (blockDim.x / SPLIT) * CP;
  const int colbase = blockIdx.z * dvp;
  const int start = P.cu_q[r], len = P.cu_q[r + 1] - start;
  if (len <= 0) return;
  const int g = h / (P.heads / P.kv_heads), G = P.kv_heads, H = P.heads;
  const int STAGE = 3 * CT * ROW + CT * dvp + CT;      // floats of one staged chunk: q, k, decay rows, values, betas
  float* os = smem + 2 * STAGE;                        // [CT][dvp]
  float* S_state = P.state + (size_t)P.state_slots[r] * P.state_stride + (size_t)h * dk * dv;
  float S[CP][DP];
  scan_state_load<CP, DP>(S, S_state, d0, colbase + col0, dk, dv);
  // the padding of both stages once: channels beyond dk (q = k = 0, decay 1) and columns beyond dv
  for (int e = threadIdx.x; e < 2 * STAGE; e += blockDim.x) {
    const int w = e % STAGE;
    smem[e] = (w >= 2 * CT * ROW && w < 3 * CT * ROW) ? 1.f : 0.f;
  }
  __syncthreads();
  auto stage = [&](int c0, int b) {
    const int nt = min(CT, len - c0), row0 = start + c0;
    float* qs = smem + b * STAGE;
    float* ks = qs + CT * ROW;
    float* gs = ks + CT * ROW;
    float* vs = gs + CT * ROW;
    float* betas = vs + CT * dvp;
    for (int e = threadIdx.x; e < nt * dk; e += blockDim.x) {
      const int i = e / dk, d = e % dk;
      const float* src = prep + (size_t)(row0 + i) * ld_prep;
      const int o = i * ROW + L::at(d);
      cp_async4(qs + o, src + (size_t)g * dk + d);
      cp_async4(ks + o, src + (size_t)(G + g) * dk + d);
      cp_async4(gs + o, src + (size_t)(2 * G + h) * dk + d);
    }
    for (int e = threadIdx.x; e < nt * dvp; e += blockDim.x) {
      const int i = e / dvp, c = e % dvp;
      if (colbase + c < dv) cp_async4(vs + e, P.v + (size_t)(row0 + i) * P.ld_qkv + (size_t)h * dv + colbase + c);
    }
    if (threadIdx.x < nt) cp_async4(betas + threadIdx.x, prep + (size_t)(row0 + threadIdx.x) * ld_prep + (size_t)(2 * G + H) * dk + h);
    cp_async_commit_group();
  };
  stage(0, 0);
  int b = 0;
  for (int c0 = 0; c0 < len; c0 += CT, b ^= 1) {
    const int nt = min(CT, len - c0), row0 = start + c0;
    if (c0 + CT < len) { stage(c0 + CT, b ^ 1); cp_async_wait_group<1>(); }
    else cp_async_wait_group<0>();
    __syncthreads();
    const float* qs = smem + b * STAGE;
    const float* ks = qs + CT * ROW;
    const float* gs = ks + CT * ROW;
    const float* vs = gs + CT * ROW;
    const float* betas = vs + CT * dvp;
    delta_tokens<L, CP, SPLIT>(S, qs, ks, gs, vs, betas, os, nt, part, col0, dvp);
    __syncthreads();
    if (E.raw) raw_out_chunk(E, os, dvp, dv, colbase, nt, row0, h);
    else head_out_chunk(E, os, dvp, dv, nt, row0, h);
    __syncthreads();       // the outputs are read, and this stage may be filled again two chunks on
  }
  scan_state_store<CP, DP>(S, S_state, d0, colbase + col0, dk, dv);
}

// ---------------------------------------------------------------------------------
// Stabilised matrix memory.
// ---------------------------------------------------------------------------------
struct MemoryIn {
  const float* q; const float* k; const float* v; long ld;       // projections [T, heads*dk], .., [T, heads*dv] (one row stride)
  const float* gi; const float* gf; long ld_gate;                // pre-activations of the input and forget gates [T, heads]
  const void* bias_i; const void* bias_f; int bias_dtype;        // [heads]
  float cap;                                                     // gates are capped: cap * tanh(z / cap)
  float* state; long state_stride;                               // per slot: S [heads, dk, dv], n [heads, dk], m [heads]
  const int* cu_q; const int* state_slots;
  int heads, dk, dv;
};

// The scalar part of the recurrence for a staged chunk, by one warp, token by token: maximum, the two factors, the
// normaliser n (a lane holds n[lane + 32 j]) and the denominator.  lf and li come in as the log gates and leave as a and b.
template <typename L, int NJ>
__device__ __forceinline__ void memory_scalars(float (&nreg)[NJ], float& m, const float* qs, const float* ks, float* li, float* lf,
                                               float* den, int nt, int lane) {
  constexpr int DK = L::DP * (L::ROW / L::STRIDE), ROW = L::ROW;
  // the scalar part of the recurrence, token by token: maximum, the two factors, normaliser and denominator
  for (int i = 0; i < nt; ++i) {
    const float f = lf[i], in = li[i];
    const float m_new = fmaxf(f + m, in);
    const float a = expf(f + m - m_new), b = expf(in - m_new);
    m = m_new;
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      const int d = lane + 32 * j;
      if (d < DK) {
        nreg[j] = fmaf(b, ks[i * ROW + L::at(d)], a * nreg[j]);
        sum = fmaf(nreg[j], qs[i * ROW + L::at(d)], sum);
      }
    }
    sum = co_warp_sum(sum);
    __syncwarp();
    if (lane == 0) { lf[i] = a; li[i] = b; den[i] = fmaxf(fabsf(sum), expf(-m)) + 1e-6f; }
  }
}

// The tokens of a staged chunk for the thread's part of S: li holds b = exp(i - m), lf holds a = exp(f + m' - m), den the
// denominators, as the scalar phase left them.
template <typename L, int CP, int SPLIT>
__device__ __forceinline__ void memory_tokens(float (&S)[CP][L::DP], const float* qs, const float* ks, const float* vs, const float* li,
                                              const float* lf, const float* den, float* os, int nt, int part, int col0, int dvp) {
  constexpr int DP = L::DP, ROW = L::ROW;
  float4 kc[DP / 4], qc[DP / 4];        // token i + 1 is fetched before token i is worked on (see the delta rule)
  scan_fetch<DP>(kc, ks + part * L::STRIDE);
  scan_fetch<DP>(qc, qs + part * L::STRIDE);
  for (int i = 0; i < nt; ++i) {
    float4 kn[DP / 4], qn[DP / 4];
    const int nx = min(i + 1, nt - 1) * ROW + part * L::STRIDE;
    scan_fetch<DP>(kn, ks + nx); scan_fetch<DP>(qn, qs + nx);
    const float a = lf[i];
    float bv[CP], o[CP][2];
#pragma unroll
    for (int c = 0; c < CP; ++c) { bv[c] = li[i] * vs[i * dvp + col0 + c]; o[c][0] = o[c][1] = 0.f; }
#pragma unroll
    for (int d = 0; d < DP / 4; ++d) {
      const float4 kk = kc[d], qq = qc[d];
#pragma unroll
      for (int c = 0; c < CP; ++c) {
        S[c][4 * d] = fmaf(bv[c], kk.x, a * S[c][4 * d]); S[c][4 * d + 1] = fmaf(bv[c], kk.y, a * S[c][4 * d + 1]);
        S[c][4 * d + 2] = fmaf(bv[c], kk.z, a * S[c][4 * d + 2]); S[c][4 * d + 3] = fmaf(bv[c], kk.w, a * S[c][4 * d + 3]);
        o[c][0] = fmaf(S[c][4 * d], qq.x, o[c][0]); o[c][1] = fmaf(S[c][4 * d + 1], qq.y, o[c][1]);
        o[c][0] = fmaf(S[c][4 * d + 2], qq.z, o[c][0]); o[c][1] = fmaf(S[c][4 * d + 3], qq.w, o[c][1]);
      }
    }
#pragma unroll
    for (int c = 0; c < CP; ++c) {
      const float y = split_sum<SPLIT>(o[c][0] + o[c][1]);
      if (part == 0) os[i * dvp + col0 + c] = y / den[i];
    }
#pragma unroll
    for (int d = 0; d < DP / 4; ++d) { kc[d] = kn[d]; qc[d] = qn[d]; }
  }
}

template <int DK, int CT, int SPLIT, int CP>
__global__ void __launch_bounds__(512) matrix_memory_scan_kernel(MemoryIn P, HeadOut E) {
  using L = ScanShape<DK, SPLIT>;
  constexpr int DP = L::DP, ROW = L::ROW;
  extern __shared__ __align__(16) float smem[];
  co_pdl_launch_dependents();
  co_pdl_wait();
  const int r = blockIdx.x, h = blockIdx.y;
  const int part = threadIdx.x % SPLIT, col0 = (threadIdx.x / SPLIT) * CP, d0 = part * DP;
  const int dk = P.dk, dv = P.dv, dvp = (blockDim.x / SPLIT) * CP;
  const int colbase = blockIdx.z * dvp;        // this CTA's first column of the head
  const int start = P.cu_q[r], len = P.cu_q[r + 1] - start;
  if (len <= 0) return;
  float* qs = smem;                    // [CT][ROW]
  float* ks = qs + CT * ROW;           // [CT][ROW]
  float* vs = ks + CT * ROW;           // [CT][dvp]
  float* os = vs + CT * dvp;           // [CT][dvp]
  float* li = os + CT * dvp;           // [CT] log input gate, then b = exp(i - m)
  float* lf = li + CT;                 // [CT] log forget gate, then a = exp(f + m' - m)
  float* den = lf + CT;                // [CT]
  float* slot = P.state + (size_t)P.state_slots[r] * P.state_stride;
  float* S_state = slot + (size_t)h * dk * dv;
  float* n_state = slot + (size_t)P.heads * dk * dv + (size_t)h * dk;
  float* m_state = slot + (size_t)P.heads * dk * dv + (size_t)P.heads * dk + h;
  float S[CP][DP];
  scan_state_load<CP, DP>(S, S_state, d0, colbase + col0, dk, dv);
  constexpr int NJ = (DK + 31) / 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float nreg[NJ];                      // warp 0: lane holds n[lane + 32 j]
  float m = 0.f;
  if (warp == 0) {
#pragma unroll
    for (int j = 0; j < NJ; ++j) nreg[j] = (lane + 32 * j < dk) ? n_state[lane + 32 * j] : 0.f;
    m = *m_state;
  }
  const float q_scale = 1.0f / sqrtf((float)dk);
  const float bi = co_load_any(P.bias_i, P.bias_dtype, h), bf = co_load_any(P.bias_f, P.bias_dtype, h);

  for (int c0 = 0; c0 < len; c0 += CT) {
    const int nt = min(CT, len - c0), row0 = start + c0;
#pragma unroll 8
    for (int e = threadIdx.x; e < nt * DK; e += blockDim.x) {      // unrolled: the loads of a thread are in flight together
      const int i = e / DK, d = e % DK;
      const size_t row = (size_t)(row0 + i);
      const int o = i * ROW + L::at(d);
      qs[o] = d < dk ? P.q[row * P.ld + (size_t)h * dk + d] * q_scale : 0.f;
      ks[o] = d < dk ? P.k[row * P.ld + (size_t)h * dk + d] : 0.f;
    }
#pragma unroll 8
    for (int e = threadIdx.x; e < nt * dvp; e += blockDim.x) {
      const int i = e / dvp, c = e % dvp;
      vs[e] = colbase + c < dv ? P.v[(size_t)(row0 + i) * P.ld + (size_t)h * dv + colbase + c] : 0.f;
    }
    if (threadIdx.x < nt) {
      const size_t row = (size_t)(row0 + threadIdx.x);
      li[threadIdx.x] = P.cap * tanhf((P.gi[row * P.ld_gate + h] + bi) / P.cap);
      const float z = P.cap * tanhf((P.gf[row * P.ld_gate + h] + bf) / P.cap);
      lf[threadIdx.x] = -rc_softplus(-z);          // log sigmoid
    }
    __syncthreads();
    if (warp == 0) memory_scalars<L, NJ>(nreg, m, qs, ks, li, lf, den, nt, lane);
    __syncthreads();
    memory_tokens<L, CP, SPLIT>(S, qs, ks, vs, li, lf, den, os, nt, part, col0, dvp);
    __syncthreads();
    if (E.raw) raw_out_chunk(E, os, dvp, dv, colbase, nt, row0, h);
    else head_out_chunk(E, os, dvp, dv, nt, row0, h);
    __syncthreads();
  }
  scan_state_store<CP, DP>(S, S_state, d0, colbase + col0, dk, dv);
  if (warp == 0 && blockIdx.z == 0) {
    // with the head's columns split over CTAs the others may not have read n and m yet: they go to the side
    float* n_to = E.nm_next ? E.nm_next + ((size_t)r * P.heads + h) * (dk + 1) : n_state;
    float* m_to = E.nm_next ? n_to + dk : m_state;
#pragma unroll
    for (int j = 0; j < NJ; ++j)
      if (lane + 32 * j < dk) n_to[lane + 32 * j] = nreg[j];
    if (lane == 0) *m_to = m;
  }
}

// For long prompts the normaliser n is kept by every thread for its own part of the key channels (beside its part of S), so
// that n . q comes out of the token loop like the columns' products and no warp walks the chunk alone first; what is left
// of the scalar part is the running maximum and the two factors of a token: lf leaves as a, li as b, em as exp(-m).
__device__ __forceinline__ void memory_factors(float& m, float* li, float* lf, float* em, int nt, int lane) {
  for (int i = 0; i < nt; ++i) {
    const float f = lf[i], in = li[i];
    const float m_new = fmaxf(f + m, in);
    const float a = expf(f + m - m_new), b = expf(in - m_new);
    m = m_new;
    __syncwarp();
    if (lane == 0) { lf[i] = a; li[i] = b; em[i] = expf(-m); }
  }
}

template <typename L, int CP, int SPLIT>
__device__ __forceinline__ void memory_tokens_n(float (&S)[CP][L::DP], float (&nn)[L::DP], const float* qs, const float* ks, const float* vs,
                                                const float* li, const float* lf, const float* em, float* os, int nt, int part,
                                                int col0, int dvp) {
  constexpr int DP = L::DP, ROW = L::ROW;
  float4 kc[DP / 4], qc[DP / 4];
  scan_fetch<DP>(kc, ks + part * L::STRIDE);
  scan_fetch<DP>(qc, qs + part * L::STRIDE);
  for (int i = 0; i < nt; ++i) {
    float4 kn[DP / 4], qn[DP / 4];
    const int nx = min(i + 1, nt - 1) * ROW + part * L::STRIDE;
    scan_fetch<DP>(kn, ks + nx); scan_fetch<DP>(qn, qs + nx);
    const float a = lf[i], b = li[i];
    float bv[CP], o[CP][2], nq0 = 0.f, nq1 = 0.f;
#pragma unroll
    for (int c = 0; c < CP; ++c) { bv[c] = b * vs[i * dvp + col0 + c]; o[c][0] = o[c][1] = 0.f; }
#pragma unroll
    for (int d = 0; d < DP / 4; ++d) {
      const float4 kk = kc[d], qq = qc[d];
      nn[4 * d] = fmaf(b, kk.x, a * nn[4 * d]); nn[4 * d + 1] = fmaf(b, kk.y, a * nn[4 * d + 1]);
      nn[4 * d + 2] = fmaf(b, kk.z, a * nn[4 * d + 2]); nn[4 * d + 3] = fmaf(b, kk.w, a * nn[4 * d + 3]);
      nq0 = fmaf(nn[4 * d], qq.x, nq0); nq1 = fmaf(nn[4 * d + 1], qq.y, nq1);
      nq0 = fmaf(nn[4 * d + 2], qq.z, nq0); nq1 = fmaf(nn[4 * d + 3], qq.w, nq1);
#pragma unroll
      for (int c = 0; c < CP; ++c) {
        S[c][4 * d] = fmaf(bv[c], kk.x, a * S[c][4 * d]); S[c][4 * d + 1] = fmaf(bv[c], kk.y, a * S[c][4 * d + 1]);
        S[c][4 * d + 2] = fmaf(bv[c], kk.z, a * S[c][4 * d + 2]); S[c][4 * d + 3] = fmaf(bv[c], kk.w, a * S[c][4 * d + 3]);
        o[c][0] = fmaf(S[c][4 * d], qq.x, o[c][0]); o[c][1] = fmaf(S[c][4 * d + 1], qq.y, o[c][1]);
        o[c][0] = fmaf(S[c][4 * d + 2], qq.z, o[c][0]); o[c][1] = fmaf(S[c][4 * d + 3], qq.w, o[c][1]);
      }
    }
    // one division per token, not one per column: the columns take the reciprocal (a last-bit difference from y / den)
    const float inv = 1.0f / (fmaxf(fabsf(split_sum<SPLIT>(nq0 + nq1)), em[i]) + 1e-6f);
#pragma unroll
    for (int c = 0; c < CP; ++c) {
      const float y = split_sum<SPLIT>(o[c][0] + o[c][1]);
      if (part == 0) os[i * dvp + col0 + c] = y * inv;
    }
#pragma unroll
    for (int d = 0; d < DP / 4; ++d) { kc[d] = kn[d]; qc[d] = qn[d]; }
  }
}

// The matrix memory for long prompts: chunks of 16 tokens staged by asynchronous copies, two deep (what is computed while
// staging is little here: q times 1 / sqrt(dk) and the two log gates of a token, done when a chunk has landed).
template <int DK, int CT, int SPLIT, int CP>
__global__ void __launch_bounds__(512) matrix_memory_scan_pre_kernel(MemoryIn P, HeadOut E) {
  using L = ScanShape<DK, SPLIT>;
  constexpr int DP = L::DP, ROW = L::ROW;
  extern __shared__ __align__(16) float smem[];
  co_pdl_launch_dependents();
  co_pdl_wait();
  const int r = blockIdx.x, h = blockIdx.y;
  const int part = threadIdx.x % SPLIT, col0 = (threadIdx.x / SPLIT) * CP, d0 = part * DP;
  const int dk = P.dk, dv = P.dv, dvp = (blockDim.x / SPLIT) * CP;
  const int colbase = blockIdx.z * dvp;
  const int start = P.cu_q[r], len = P.cu_q[r + 1] - start;
  if (len <= 0) return;
  const int STAGE = 2 * CT * ROW + CT * dvp + 2 * CT;      // floats of one staged chunk: q, k rows, values, the two gates
  float* os = smem + 2 * STAGE;                            // [CT][dvp]
  float* den = os + CT * dvp;                              // [CT]
  float* slot = P.state + (size_t)P.state_slots[r] * P.state_stride;
  float* S_state = slot + (size_t)h * dk * dv;
  float* n_state = slot + (size_t)P.heads * dk * dv + (size_t)h * dk;
  float* m_state = slot + (size_t)P.heads * dk * dv + (size_t)P.heads * dk + h;
  float S[CP][DP];
  scan_state_load<CP, DP>(S, S_state, d0, colbase + col0, dk, dv);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float nn[DP];                        // this thread's part of the normaliser
#pragma unroll
  for (int d = 0; d < DP; ++d) nn[d] = d0 + d < dk ? n_state[d0 + d] : 0.f;
  float m = warp == 0 ? *m_state : 0.f;
  const float q_scale = 1.0f / sqrtf((float)dk);
  const float bi = co_load_any(P.bias_i, P.bias_dtype, h), bf = co_load_any(P.bias_f, P.bias_dtype, h);
  for (int e = threadIdx.x; e < 2 * STAGE; e += blockDim.x) smem[e] = 0.f;      // the padding of both stages, once
  __syncthreads();
  auto stage = [&](int c0, int b) {
    const int nt = min(CT, len - c0), row0 = start + c0;
    float* qs = smem + b * STAGE;
    float* ks = qs + CT * ROW;
    float* vs = ks + CT * ROW;
    float* gates = vs + CT * dvp;
    for (int e = threadIdx.x; e < nt * dk; e += blockDim.x) {
      const int i = e / dk, d = e % dk;
      const size_t row = (size_t)(row0 + i);
      const int o = i * ROW + L::at(d);
      cp_async4(qs + o, P.q + row * P.ld + (size_t)h * dk + d);
      cp_async4(ks + o, P.k + row * P.ld + (size_t)h * dk + d);
    }
    for (int e = threadIdx.x; e < nt * dvp; e += blockDim.x) {
      const int i = e / dvp, c = e % dvp;
      if (colbase + c < dv) cp_async4(vs + e, P.v + (size_t)(row0 + i) * P.ld + (size_t)h * dv + colbase + c);
    }
    if (threadIdx.x < nt) {
      cp_async4(gates + threadIdx.x, P.gi + (size_t)(row0 + threadIdx.x) * P.ld_gate + h);
      cp_async4(gates + CT + threadIdx.x, P.gf + (size_t)(row0 + threadIdx.x) * P.ld_gate + h);
    }
    cp_async_commit_group();
  };
  stage(0, 0);
  int b = 0;
  for (int c0 = 0; c0 < len; c0 += CT, b ^= 1) {
    const int nt = min(CT, len - c0), row0 = start + c0;
    if (c0 + CT < len) { stage(c0 + CT, b ^ 1); cp_async_wait_group<1>(); }
    else cp_async_wait_group<0>();
    __syncthreads();
    float* qs = smem + b * STAGE;
    float* ks = qs + CT * ROW;
    float* vs = ks + CT * ROW;
    float* li = vs + CT * dvp;
    float* lf = li + CT;
    for (int e = threadIdx.x; e < nt * dk; e += blockDim.x) qs[(e / dk) * ROW + L::at(e % dk)] *= q_scale;
    if (threadIdx.x < nt) {
      li[threadIdx.x] = P.cap * tanhf((li[threadIdx.x] + bi) / P.cap);
      const float z = P.cap * tanhf((lf[threadIdx.x] + bf) / P.cap);
      lf[threadIdx.x] = -rc_softplus(-z);
    }
    __syncthreads();
    if (warp == 0) memory_factors(m, li, lf, den, nt, lane);
    __syncthreads();
    memory_tokens_n<L, CP, SPLIT>(S, nn, qs, ks, vs, li, lf, den, os, nt, part, col0, dvp);
    __syncthreads();
    if (E.raw) raw_out_chunk(E, os, dvp, dv, colbase, nt, row0, h);
    else head_out_chunk(E, os, dvp, dv, nt, row0, h);
    __syncthreads();
  }
  scan_state_store<CP, DP>(S, S_state, d0, colbase + col0, dk, dv);
  if (blockIdx.z == 0 && threadIdx.x < SPLIT) {      // the first group of lanes holds the whole of n between them
    float* n_to = E.nm_next ? E.nm_next + ((size_t)r * P.heads + h) * (dk + 1) : n_state;
    float* m_to = E.nm_next ? n_to + dk : m_state;
#pragma unroll
    for (int d = 0; d < DP; ++d)
      if (d0 + d < dk) n_to[d0 + d] = nn[d];
    if (threadIdx.x == 0) *m_to = m;
  }
}

// ---------------------------------------------------------------------------------
// Queries and keys normalised over the WHOLE projection (all heads at once), keys and values written into
// cache pages: q_out[t] = q / rms(q) * wq, K[slot] = k / rms(k) * wk, V[slot] = v.  A CTA per token.
// normalise = 0 copies q and k as they are.  v_scale multiplies the values (an attention whose output is
// multiplied by a constant can keep its values multiplied instead).
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
qk_norm_kv_write_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, long ld,
                        const void* __restrict__ wq, const void* __restrict__ wk, int w_dtype, float eps, int normalise,
                        T* __restrict__ q_out, long ldq, const int* __restrict__ slots, T* __restrict__ k_cache,
                        T* __restrict__ v_cache, int nh, int nkv, int dk, int dv, int page_size, float v_scale) {
  __shared__ float scratch[33];
  co_pdl_launch_dependents();
  co_pdl_wait();
  const size_t t = blockIdx.x;
  const int nq = nh * dk, nk = nkv * dk, nv = nkv * dv;
  const float* qr = q + t * ld;
  const float* kr = k + t * ld;
  const float* vr = v + t * ld;
  float iq = 1.f, ik = 1.f;
  if (normalise) {
    float s = 0.f;
    for (int e = threadIdx.x; e < nq; e += blockDim.x) s = fmaf(qr[e], qr[e], s);
    iq = 1.0f / sqrtf(co_block_sum(s, scratch) / (float)nq + eps);
    s = 0.f;
    for (int e = threadIdx.x; e < nk; e += blockDim.x) s = fmaf(kr[e], kr[e], s);
    ik = 1.0f / sqrtf(co_block_sum(s, scratch) / (float)nk + eps);
  }
  for (int e = threadIdx.x; e < nq; e += blockDim.x)
    q_out[t * ldq + e] = co_from_float<T>(normalise ? qr[e] * iq * co_load_any(wq, w_dtype, e) : qr[e]);
  if (!slots) return;
  const int slot = slots[t];
  const size_t page = slot / page_size, off = slot % page_size;
  for (int e = threadIdx.x; e < nk; e += blockDim.x) {
    const int g = e / dk, d = e % dk;
    k_cache[((page * nkv + g) * page_size + off) * dk + d] =
        co_from_float<T>(normalise ? kr[e] * ik * co_load_any(wk, w_dtype, e) : kr[e]);
  }
  for (int e = threadIdx.x; e < nv; e += blockDim.x) {
    const int g = e / dv, d = e % dv;
    v_cache[((page * nkv + g) * page_size + off) * dv + d] = co_from_float<T>(vr[e] * v_scale);
  }
}

constexpr int chunk_tokens(int DK) { return DK <= 128 ? 32 : 16; }
// Lanes per group of columns and columns per group.  The more lanes share a column, the fewer steps a token costs
// each of them (the recurrence is a chain of dependent steps, and that chain is what bounds a long prompt): sixteen
// from 128 key channels on, eight from 64, four below.  Four columns per group (two for narrow heads); a head of more
// than 128 value channels takes twice as many so that the CTA stays within 512 threads.
constexpr int scan_split(int DK) { return DK >= 128 ? 16 : (DK >= 64 ? 8 : 4); }
constexpr int scan_columns(int DK, bool wide) { return (DK >= 64 ? 4 : 2) * (wide ? 2 : 1); }

}  // namespace

CO_EXPORT int coheryn_short_conv_silu(const float* x, long ldx, float* y, long ldy, const void* taps, int taps_dtype, int n,
                                      int C, float* state, long state_stride, const int* token_req, const int* cu_q,
                                      const int* state_slots, int T, int B, int update_state, cudaStream_t stream) {
  if (T <= 0 || C <= 0) return 0;
  if (n < 1 || n > MAX_TAPS) CO_FAIL("short_conv: 1..%d taps, not %d", MAX_TAPS, n);
  const size_t total = (size_t)T * C;
  co_launch(short_conv_silu_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, x, ldx, y, ldy, taps, taps_dtype, n,
            C, (const float*)state, state_stride, token_req, cu_q, state_slots, T);
  CO_CHECK_LAUNCH("short_conv_silu");
  if (update_state && n > 1) {
    const size_t per = (size_t)B * C;
    co_launch(short_conv_state_kernel, dim3((unsigned)((per + 255) / 256)), dim3(256), 0, stream, x, ldx, n, C, state, state_stride,
              cu_q, state_slots, B);
    CO_CHECK_LAUNCH("short_conv_state");
  }
  return 0;
}

#define CO_SCAN_CASES(LAUNCH)                                                                   \
  if (dk <= 16) { LAUNCH(16) } else if (dk <= 32) { LAUNCH(32) } else if (dk <= 48) { LAUNCH(48) } \
  else if (dk <= 64) { LAUNCH(64) } else if (dk <= 96) { LAUNCH(96) } else if (dk <= 128) { LAUNCH(128) } \
  else if (dk <= 192) { LAUNCH(192) } else { LAUNCH(256) }

// Into how many CTAs the columns of a head are split: one (the scan's own epilogue normalises whole heads) unless the
// step is a long prompt of few requests, where a CTA per head would leave most SMs idle; then 64 columns per CTA, the
// unnormalised outputs in the caller's scratch (total_tokens * heads * dv floats, then `extra`) and the norm in a kernel
// of its own.  A column's arithmetic is the same either way.
constexpr int SLICE_COLUMNS = 64;
static int scan_slices(int B, int heads, int dv, int total_tokens, const float* scratch, long scratch_floats, long extra) {
  if (!scratch || dv <= SLICE_COLUMNS || (long)B * heads > 74 || total_tokens < 64 * B) return 1;
  if (scratch_floats < (long)total_tokens * heads * dv + extra) return 1;
  return (dv + SLICE_COLUMNS - 1) / SLICE_COLUMNS;
}

static int launch_head_norm_gate(const HeadOut& E, int T, int heads, int dv, cudaStream_t stream) {
  const size_t smem = (size_t)16 * dv * sizeof(float);
  co_launch(head_norm_gate_kernel, dim3((T + 15) / 16, heads), dim3(256), smem, stream, E, T, dv);
  CO_CHECK_LAUNCH("head_norm_gate");
  return 0;
}

static int scan_shape_ok(const char* name, int heads, int dk, int dv) {
  if (heads < 1 || dk < 1 || dk > 256 || dv < 1 || dv > 256) {
    co_set_error("%s: heads %d, key channels %d (1..256), value channels %d (1..256)", name, heads, dk, dv);
    return 0;
  }
  return 1;
}

CO_EXPORT int coheryn_gated_delta_scan(
    const float* q, const float* k, const float* v, long ld_qkv, const float* beta, long ld_beta, const float* step,
    long ld_step, const void* step_bias, int step_bias_dtype, const void* rate_log, int rate_log_dtype, float* state,
    long state_stride, const int* cu_q, const int* state_slots, int B, int heads, int kv_heads, int dk, int dv, void* out,
    int out_dtype, long ldo, const void* weight, int weight_dtype, int weight_stride, const float* gate, long ldg, float eps,
    float out_scale, int total_tokens, float* scratch, long scratch_floats, int decay_channels, int gate_act,
    cudaStream_t stream) {
  if (B <= 0) return 0;
  if (!scan_shape_ok("gated_delta_scan", heads, dk, dv)) return 1;
  if (decay_channels != 1 && decay_channels != dk) CO_FAIL("gated_delta_scan: a decay per head (1) or per key channel (%d), not %d", dk, decay_channels);
  if (gate_act != 0 && gate_act != 1) CO_FAIL("gated_delta_scan: unknown gate activation %d", gate_act);
  const long ld_prep = (long)2 * kv_heads * dk + (long)heads * dk + heads;     // per token: q, k, decays, beta
  const int slices = scan_slices(B, heads, dv, total_tokens, scratch, scratch_floats, (long)total_tokens * ld_prep);
  float* prep = slices > 1 ? scratch + (long)total_tokens * heads * dv : nullptr;
  if (kv_heads < 1 || heads % kv_heads) CO_FAIL("gated_delta_scan: %d heads do not group over %d q/k heads", heads, kv_heads);
  DeltaIn P{q, k, v, ld_qkv, beta, ld_beta, step, ld_step, step_bias, step_bias_dtype, rate_log, rate_log_dtype, state,
            state_stride, cu_q, state_slots, heads, kv_heads, dk, dv, decay_channels};
  HeadOut E{out, out_dtype, ldo, weight, weight_dtype, weight_stride, gate, ldg, eps, out_scale,
            slices > 1 ? scratch : nullptr, (long)heads * dv, nullptr, gate_act};
  if (slices > 1) {
    co_launch(delta_prepare_kernel, dim3(total_tokens), dim3(128), 0, stream, P, prep, ld_prep);
    CO_CHECK_LAUNCH("delta_prepare");
  }
#define LAUNCH_CP(D, WIDE)                                                                                     \
  {                                                                                                            \
    constexpr int CT = chunk_tokens(D), SP = scan_split(D), CP = scan_columns(D, WIDE), ROW = ScanShape<D, SP>::ROW; \
    const int cols = slices > 1 ? SLICE_COLUMNS : dv;                                                          \
    const int threads = ((cols + CP - 1) / CP * SP + 31) / 32 * 32, dvp = threads / SP * CP;                   \
    if (slices > 1) {   /* a long prompt: prepared inputs, asynchronous staging of 16 tokens, two deep */          \
      constexpr int CA = 16;                                                                                   \
      const size_t smem = ((size_t)2 * (3 * CA * ROW + CA * dvp + CA) + (size_t)CA * dvp) * sizeof(float);     \
      auto kern = gated_delta_scan_pre_kernel<D, CA, SP, CP>;                                                  \
      if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      co_launch_ex(true, kern, dim3(B, heads, (dv + dvp - 1) / dvp), dim3(threads), smem, stream, P, E, (const float*)prep, ld_prep); \
    } else {                                                                                                   \
      const size_t smem = ((size_t)3 * CT * ROW + (size_t)2 * CT * dvp + CT) * sizeof(float);                  \
      auto kern = gated_delta_scan_kernel<D, CT, SP, CP>;                                                      \
      if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      co_launch_ex(true, kern, dim3(B, heads, 1), dim3(threads), smem, stream, P, E);                          \
    }                                                                                                          \
  }
#define LAUNCH(D) if (slices == 1 && dv * scan_split(D) > 128 * 16) LAUNCH_CP(D, true) else LAUNCH_CP(D, false)
  CO_SCAN_CASES(LAUNCH)
#undef LAUNCH
#undef LAUNCH_CP
  CO_CHECK_LAUNCH("gated_delta_scan");
  return slices > 1 ? launch_head_norm_gate(E, total_tokens, heads, dv, stream) : 0;
}

CO_EXPORT int coheryn_matrix_memory_scan(
    const float* q, const float* k, const float* v, long ld, const float* gi, const float* gf, long ld_gate,
    const void* bias_i, const void* bias_f, int bias_dtype, float cap, float* state, long state_stride, const int* cu_q,
    const int* state_slots, int B, int heads, int dk, int dv, void* out, int out_dtype, long ldo, const void* weight,
    int weight_dtype, int weight_stride, const float* gate, long ldg, float eps, float out_scale, int total_tokens,
    float* scratch, long scratch_floats, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (!scan_shape_ok("matrix_memory_scan", heads, dk, dv)) return 1;
  const int slices = scan_slices(B, heads, dv, total_tokens, scratch, scratch_floats, (long)B * heads * (dk + 1));
  if (!(cap > 0.f)) CO_FAIL("matrix_memory_scan: the gate cap must be positive");
  MemoryIn P{q, k, v, ld, gi, gf, ld_gate, bias_i, bias_f, bias_dtype, cap, state, state_stride, cu_q, state_slots, heads, dk, dv};
  HeadOut E{out, out_dtype, ldo, weight, weight_dtype, weight_stride, gate, ldg, eps, out_scale,
            slices > 1 ? scratch : nullptr, (long)heads * dv, slices > 1 ? scratch + (long)total_tokens * heads * dv : nullptr};
#define LAUNCH_CP(D, WIDE)                                                                                     \
  {                                                                                                            \
    constexpr int CT = chunk_tokens(D), SP = scan_split(D), CP = scan_columns(D, WIDE), ROW = ScanShape<D, SP>::ROW; \
    const int cols = slices > 1 ? SLICE_COLUMNS : dv;                                                          \
    const int threads = ((cols + CP - 1) / CP * SP + 31) / 32 * 32, dvp = threads / SP * CP;                   \
    if (slices > 1) {   /* a long prompt: asynchronous staging of 16 tokens, two deep */                        \
      constexpr int CA = 16;                                                                                   \
      const size_t smem = ((size_t)2 * (2 * CA * ROW + CA * dvp + 2 * CA) + (size_t)CA * dvp + CA) * sizeof(float); \
      auto kern = matrix_memory_scan_pre_kernel<D, CA, SP, CP>;                                                \
      if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      co_launch_ex(true, kern, dim3(B, heads, (dv + dvp - 1) / dvp), dim3(threads), smem, stream, P, E);       \
    } else {                                                                                                   \
      const size_t smem = ((size_t)2 * CT * ROW + (size_t)2 * CT * dvp + 3 * CT) * sizeof(float);              \
      auto kern = matrix_memory_scan_kernel<D, CT, SP, CP>;                                                    \
      if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      co_launch_ex(true, kern, dim3(B, heads, 1), dim3(threads), smem, stream, P, E);                          \
    }                                                                                                          \
  }
#define LAUNCH(D) if (slices == 1 && dv * scan_split(D) > 128 * 16) LAUNCH_CP(D, true) else LAUNCH_CP(D, false)
  CO_SCAN_CASES(LAUNCH)
#undef LAUNCH
#undef LAUNCH_CP
  CO_CHECK_LAUNCH("matrix_memory_scan");
  if (slices == 1) return 0;
  co_launch(memory_nm_commit_kernel, dim3(B, heads), dim3(128), 0, stream, (const float*)E.nm_next, state, state_stride, state_slots,
            cu_q, heads, dk, dv);
  CO_CHECK_LAUNCH("memory_nm_commit");
  return launch_head_norm_gate(E, total_tokens, heads, dv, stream);
}

CO_EXPORT int coheryn_qk_norm_kv_write(const float* q, const float* k, const float* v, long ld, const void* wq, const void* wk,
                                       int w_dtype, float eps, int normalise, void* q_out, int dtype, long ldq, const int* slots,
                                       void* k_cache, void* v_cache, int T, int nh, int nkv, int dk, int dv, int page_size,
                                       float v_scale, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (nh < 1 || nkv < 0 || dk < 1 || dv < 1 || page_size < 1) CO_FAIL("qk_norm_kv_write: bad sizes");
  if (dtype == CO_F32)
    co_launch(qk_norm_kv_write_kernel<float>, dim3(T), dim3(256), 0, stream, q, k, v, ld, wq, wk, w_dtype, eps, normalise,
              (float*)q_out, ldq, slots, (float*)k_cache, (float*)v_cache, nh, nkv, dk, dv, page_size, v_scale);
  else if (dtype == CO_BF16)
    co_launch(qk_norm_kv_write_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, q, k, v, ld, wq, wk, w_dtype, eps, normalise,
              (__nv_bfloat16*)q_out, ldq, slots, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, nh, nkv, dk, dv, page_size,
              v_scale);
  else
    CO_FAIL("qk_norm_kv_write: unknown dtype %d", dtype);
  CO_CHECK_LAUNCH("qk_norm_kv_write");
  return 0;
}
