// Sequence-mixer kernels for hybrid decoders on sm_100a: recurrent (linear-attention / delta-rule) layers with a fixed-size
// fp32 state per sequence, short causal convolutions with a carried window, and paged attention with a learned
// distance-bucket bias and an optional softmax sink.  All of them work on a RAGGED step: the flat token batch holds, for
// every live sequence, the next `q_len` tokens (a whole prompt, a portion of one, or one decoded token), described by
//
//   cu_q[nseq + 1]   first flat token index of every sequence's portion
//   ctx_len[nseq]    tokens of the sequence that earlier steps already consumed (0 = a fresh sequence: the carried state
//                    is taken as zero, so a recycled slot needs no clearing)
//   slots[nseq]      index of the sequence's state slot in the per-layer state pool
//
// Every recurrence runs token by token in fp32 with one fixed order of operations, so the result at a position does not
// depend on how the prompt was cut or on what else is in the batch.
//
//   cb_short_conv_silu      y = silu(causal depthwise conv(x)) over time, window of taps-1 inputs carried per slot
//   cb_state_scan           S <- decay * S + k (x) v   (scalar decay per head), or the gated delta rule
//                           S <- g * S; u = beta (v - S^T k); S <- S + k (x) u  (decay per key channel); o = S^T q
//   cb_gated_group_rmsnorm  out = o / rms_group(o) * w * sigmoid(gate)
//   cb_rmsnorm_residual     x(fp32) += mult * y / rms(y) * (offset + w);  h = cast(x)
//   cb_rmsnorm_f32in        out = cast(x / rms(x) * (offset + w)) for an fp32 residual stream
//   cb_paged_kv_write_mix   K / V rows (different widths allowed) into the paged cache, V optionally blended with another
//                           layer's values first
//   cb_paged_bias_attention causal attention of every step token over its sequence's paged cache with
//                           score = scale * q.k + table[bucket(distance)][head] and an optional zero-score sink
#include "common.cuh"

namespace {

CB_DEVICE float silu_f(float x) { return x / (1.f + expf(-x)); }
CB_DEVICE float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
CB_DEVICE float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// ------------------------------------------------------------------------------------------------ short convolution
constexpr int CONV_MAX_TAPS = 8;
constexpr int CONV_TOK_TILE = 32;

template <typename T>
__global__ void __launch_bounds__(128) short_conv_silu_kernel(const T* __restrict__ x, int64_t ldx, const T* __restrict__ w,
                                                              const T* __restrict__ state, T* __restrict__ out,
                                                              int64_t ldo, const int* __restrict__ cu_q,
                                                              const int* __restrict__ ctx_len,
                                                              const int* __restrict__ slots, int C, int taps,
                                                              int apply_silu) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int s = blockIdx.z;
  const int t0 = cu_q[s], qlen = cu_q[s + 1] - t0;
  const int j0 = blockIdx.y * CONV_TOK_TILE;
  if (c >= C || j0 >= qlen) return;
  const bool carried = ctx_len[s] > 0;
  const T* st = state + (int64_t)slots[s] * (taps - 1) * C;
  float wt[CONV_MAX_TAPS], win[CONV_MAX_TAPS];
#pragma unroll
  for (int i = 0; i < CONV_MAX_TAPS; ++i) {
    wt[i] = i < taps ? to_f32<T>(w[(int64_t)c * taps + i]) : 0.f;
    win[i] = 0.f;
    if (i < taps - 1) {
      const int rel = j0 - (taps - 1) + i;
      if (rel >= 0) win[i] = to_f32<T>(x[(int64_t)(t0 + rel) * ldx + c]);
      else if (carried) win[i] = to_f32<T>(st[(int64_t)(taps - 1 + rel) * C + c]);
    }
  }
  const int j1 = min(j0 + CONV_TOK_TILE, qlen);
  for (int j = j0; j < j1; ++j) {
    const float cur = to_f32<T>(x[(int64_t)(t0 + j) * ldx + c]);
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < CONV_MAX_TAPS - 1; ++i)
      if (i < taps - 1) acc = fmaf(wt[i], win[i], acc);
#pragma unroll
    for (int i = 0; i < CONV_MAX_TAPS; ++i)
      if (i == taps - 1) acc = fmaf(wt[i], cur, acc);
    out[(int64_t)(t0 + j) * ldo + c] = from_f32<T>(apply_silu ? silu_f(acc) : acc);
#pragma unroll
    for (int i = 0; i < CONV_MAX_TAPS - 1; ++i) {
      if (i < taps - 2) win[i] = win[i + 1];
      else if (i == taps - 2) win[i] = cur;
    }
  }
}

// the window a later step starts from: the last taps-1 inputs of the sequence (older ones come from the old window
// when the portion is shorter than that); every thread reads all it needs before it writes
template <typename T>
__global__ void __launch_bounds__(128) short_conv_state_kernel(const T* __restrict__ x, int64_t ldx, T* __restrict__ state,
                                                               const int* __restrict__ cu_q,
                                                               const int* __restrict__ ctx_len,
                                                               const int* __restrict__ slots, int C, int taps) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int s = blockIdx.y;
  const int t0 = cu_q[s], qlen = cu_q[s + 1] - t0;
  if (c >= C || qlen == 0) return;
  const bool carried = ctx_len[s] > 0;
  T* st = state + (int64_t)slots[s] * (taps - 1) * C;
  T val[CONV_MAX_TAPS];
#pragma unroll
  for (int i = 0; i < CONV_MAX_TAPS - 1; ++i) {
    val[i] = from_f32<T>(0.f);
    if (i < taps - 1) {
      const int rel = qlen - (taps - 1) + i;
      if (rel >= 0) val[i] = x[(int64_t)(t0 + rel) * ldx + c];
      else if (carried) val[i] = st[(int64_t)(taps - 1 + rel) * C + c];
    }
  }
#pragma unroll
  for (int i = 0; i < CONV_MAX_TAPS - 1; ++i)
    if (i < taps - 1) st[(int64_t)i * C + c] = val[i];
}

// ------------------------------------------------------------------------------------------------ recurrent state scan
enum ScanMode : int { SCAN_DECAY = 0, SCAN_DELTA = 1 };
constexpr int SCAN_TOK_TILE = 16;

struct ScanParams {
  const void *q, *k, *v;        // [T, ld*]: q/k hold qk_heads x dim, v holds heads x vdim
  int64_t ldq, ldk, ldv;
  const void* araw;             // delta: pre-activation of the decay [T, lda] (heads x dim)
  int64_t lda;
  const void* braw;             // delta: pre-activation of the write strength [T, ldb] (heads)
  int64_t ldb;
  const float* head_decay;      // decay mode: [heads]
  const float* a_log;           // delta: [heads]
  const float* dt_bias;         // delta: [heads x dim]
  float* state;                 // [slots, heads, dim, vdim] fp32
  float* out;                   // [T, heads x vdim] fp32
  const int *cu_q, *ctx_len, *slots;
  int heads, qk_heads, dim, vdim;
  int act_silu;                 // silu on q, k, v when they are loaded
  int unit_qk;                  // q, k divided by sqrt(sum x^2 + unit_eps) per head
  float unit_eps, q_scale;
};

template <int DK, int MODE, typename T>
__global__ void __launch_bounds__(128) state_scan_kernel(ScanParams p) {
  __shared__ __align__(16) float sq[SCAN_TOK_TILE][DK];
  __shared__ __align__(16) float sk[SCAN_TOK_TILE][DK];
  __shared__ __align__(16) float sg[MODE == SCAN_DELTA ? SCAN_TOK_TILE : 1][DK];
  __shared__ float sbeta[SCAN_TOK_TILE];
  const int vblocks = (p.vdim + blockDim.x - 1) / blockDim.x;
  const int h = blockIdx.x / vblocks, vb = blockIdx.x % vblocks;
  const int s = blockIdx.y;
  const int t0 = p.cu_q[s], t1 = p.cu_q[s + 1];
  if (t0 >= t1) return;
  const int j = vb * blockDim.x + threadIdx.x;
  const bool active = j < p.vdim;
  const int hk = h / (p.heads / p.qk_heads);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int dim = p.dim, vdim = p.vdim;
  float* Sg = p.state + ((int64_t)p.slots[s] * p.heads + h) * dim * vdim;
  float S[DK];
  const bool carried = p.ctx_len[s] > 0;
#pragma unroll
  for (int i = 0; i < DK; ++i) S[i] = (carried && active && i < dim) ? Sg[(int64_t)i * vdim + j] : 0.f;
  const T* q = (const T*)p.q;
  const T* k = (const T*)p.k;
  const T* v = (const T*)p.v;
  const float hd = MODE == SCAN_DECAY ? p.head_decay[h] : 0.f;
  const float A = MODE == SCAN_DELTA ? expf(p.a_log[h]) : 0.f;

  for (int tb = t0; tb < t1; tb += SCAN_TOK_TILE) {
    const int nt = min(SCAN_TOK_TILE, t1 - tb);
    __syncthreads();
    for (int tt = warp; tt < nt; tt += nwarps) {
      const int64_t t = tb + tt;
      float ssq = 0.f, ssk = 0.f;
      for (int i = lane; i < DK; i += 32) {
        float qv = 0.f, kv = 0.f;
        if (i < dim) {
          qv = to_f32<T>(q[t * p.ldq + hk * dim + i]);
          kv = to_f32<T>(k[t * p.ldk + hk * dim + i]);
          if (p.act_silu) { qv = silu_f(qv); kv = silu_f(kv); }
        }
        ssq = fmaf(qv, qv, ssq);
        ssk = fmaf(kv, kv, ssk);
        sq[tt][i] = qv;
        sk[tt][i] = kv;
        if (MODE == SCAN_DELTA) {
          float g = 1.f;
          if (i < dim) {
            const float a = to_f32<T>(((const T*)p.araw)[t * p.lda + h * dim + i]) + p.dt_bias[h * dim + i];
            g = expf(-A * softplus_f(a));
          }
          sg[tt][i] = g;
        }
      }
      float rq = p.q_scale, rk = 1.f;
      if (p.unit_qk) {
        ssq = warp_sum(ssq);
        ssk = warp_sum(ssk);
        rq = p.q_scale / sqrtf(ssq + p.unit_eps);
        rk = 1.f / sqrtf(ssk + p.unit_eps);
      }
      for (int i = lane; i < DK; i += 32) {   // a lane rescales what it wrote itself
        sq[tt][i] *= rq;
        sk[tt][i] *= rk;
      }
      if (MODE == SCAN_DELTA && lane == 0) sbeta[tt] = sigmoid_f(to_f32<T>(((const T*)p.braw)[t * p.ldb + h]));
    }
    __syncthreads();
    if (!active) continue;
    for (int tt = 0; tt < nt; ++tt) {
      const int64_t t = tb + tt;
      float vv = to_f32<T>(v[t * p.ldv + h * vdim + j]);
      if (p.act_silu) vv = silu_f(vv);
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
      if (MODE == SCAN_DELTA) {
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
        for (int i = 0; i < DK; i += 4) {
          const float4 g4 = *reinterpret_cast<const float4*>(&sg[tt][i]);
          const float4 k4 = *reinterpret_cast<const float4*>(&sk[tt][i]);
          S[i] *= g4.x; S[i + 1] *= g4.y; S[i + 2] *= g4.z; S[i + 3] *= g4.w;
          a0 = fmaf(S[i], k4.x, a0); a1 = fmaf(S[i + 1], k4.y, a1);
          a2 = fmaf(S[i + 2], k4.z, a2); a3 = fmaf(S[i + 3], k4.w, a3);
        }
        const float u = sbeta[tt] * (vv - ((a0 + a1) + (a2 + a3)));
#pragma unroll
        for (int i = 0; i < DK; i += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(&sk[tt][i]);
          const float4 q4 = *reinterpret_cast<const float4*>(&sq[tt][i]);
          S[i] = fmaf(k4.x, u, S[i]); S[i + 1] = fmaf(k4.y, u, S[i + 1]);
          S[i + 2] = fmaf(k4.z, u, S[i + 2]); S[i + 3] = fmaf(k4.w, u, S[i + 3]);
          o0 = fmaf(S[i], q4.x, o0); o1 = fmaf(S[i + 1], q4.y, o1);
          o2 = fmaf(S[i + 2], q4.z, o2); o3 = fmaf(S[i + 3], q4.w, o3);
        }
      } else {
#pragma unroll
        for (int i = 0; i < DK; i += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(&sk[tt][i]);
          const float4 q4 = *reinterpret_cast<const float4*>(&sq[tt][i]);
          S[i] = fmaf(hd, S[i], k4.x * vv); S[i + 1] = fmaf(hd, S[i + 1], k4.y * vv);
          S[i + 2] = fmaf(hd, S[i + 2], k4.z * vv); S[i + 3] = fmaf(hd, S[i + 3], k4.w * vv);
          o0 = fmaf(S[i], q4.x, o0); o1 = fmaf(S[i + 1], q4.y, o1);
          o2 = fmaf(S[i + 2], q4.z, o2); o3 = fmaf(S[i + 3], q4.w, o3);
        }
      }
      p.out[t * ((int64_t)p.heads * vdim) + h * vdim + j] = (o0 + o1) + (o2 + o3);
    }
  }
  if (active) {
#pragma unroll
    for (int i = 0; i < DK; ++i)
      if (i < dim) Sg[(int64_t)i * vdim + j] = S[i];
  }
}

template <int MODE, typename T> int launch_scan(const ScanParams& p, int nseq, cudaStream_t st) {
  int threads = ((p.vdim + 31) / 32) * 32;
  if (threads > 128) threads = 128;
  const int vblocks = (p.vdim + threads - 1) / threads;
  dim3 grid(p.heads * vblocks, nseq);
  if (p.dim <= 16) state_scan_kernel<16, MODE, T><<<grid, threads, 0, st>>>(p);
  else if (p.dim <= 32) state_scan_kernel<32, MODE, T><<<grid, threads, 0, st>>>(p);
  else if (p.dim <= 64) state_scan_kernel<64, MODE, T><<<grid, threads, 0, st>>>(p);
  else if (p.dim <= 128) state_scan_kernel<128, MODE, T><<<grid, threads, 0, st>>>(p);
  else return (int)cudaErrorInvalidValue;
  return CB_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------------------ norms
// one warp per (token, group): out = o / sqrt(mean_group(o^2) + eps) * w[c % wn] * sigmoid(gate)
template <typename T>
__global__ void __launch_bounds__(256) gated_group_rmsnorm_kernel(const float* __restrict__ o, const T* __restrict__ w,
                                                                  int wn, const T* __restrict__ gate, int64_t ldg,
                                                                  T* __restrict__ out, int64_t tokens, int C, int group,
                                                                  float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t unit = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int ngroups = C / group;
  if (unit >= tokens * ngroups) return;
  const int64_t t = unit / ngroups;
  const int c0 = (int)(unit % ngroups) * group;
  const float* row = o + t * C + c0;
  float ss = 0.f;
  for (int i = lane; i < group; i += 32) ss = fmaf(row[i], row[i], ss);
  ss = warp_sum(ss);
  const float r = 1.f / sqrtf(ss / (float)group + eps);
  for (int i = lane; i < group; i += 32) {
    const int c = c0 + i;
    float y = row[i] * r * to_f32<T>(w[c % wn]);
    if (gate != nullptr) y *= sigmoid_f(to_f32<T>(gate[t * ldg + c]));
    out[t * C + c] = from_f32<T>(y);
  }
}

// one CTA per token row.  x (fp32) += mult * y / rms(y) * (offset + w); h = cast(x)
template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_residual_kernel(float* __restrict__ x, const T* __restrict__ y, int64_t ldy,
                                                               const T* __restrict__ w, T* __restrict__ h, int W,
                                                               float eps, float mult, float offset) {
  __shared__ float red[64];
  const int64_t t = blockIdx.x;
  const T* yr = y + t * ldy;
  float ss[1] = {0.f};
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float a = to_f32<T>(yr[i]);
    ss[0] = fmaf(a, a, ss[0]);
  }
  block_sum<1>(ss, red);
  const float r = 1.f / sqrtf(ss[0] / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float nx = x[t * W + i] + mult * (to_f32<T>(yr[i]) * r * (offset + to_f32<T>(w[i])));
    x[t * W + i] = nx;
    if (h != nullptr) h[t * W + i] = from_f32<T>(nx);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_f32in_kernel(const float* __restrict__ x, const T* __restrict__ w,
                                                            T* __restrict__ out, int W, float eps, float offset) {
  __shared__ float red[64];
  const int64_t t = blockIdx.x;
  float ss[1] = {0.f};
  for (int i = threadIdx.x; i < W; i += blockDim.x) ss[0] = fmaf(x[t * W + i], x[t * W + i], ss[0]);
  block_sum<1>(ss, red);
  const float r = 1.f / sqrtf(ss[0] / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x)
    out[t * W + i] = from_f32<T>(x[t * W + i] * r * (offset + to_f32<T>(w[i])));
}

// ------------------------------------------------------------------------------------------------ paged cache write
template <typename T>
__global__ void __launch_bounds__(128) paged_kv_write_mix_kernel(const T* __restrict__ k, int64_t ldk, const T* __restrict__ v,
                                                                 int64_t ldv, const T* __restrict__ v_other,
                                                                 int64_t ldvo, float lam, T* __restrict__ k_cache,
                                                                 T* __restrict__ v_cache,
                                                                 const int* __restrict__ block_tables,
                                                                 const int* __restrict__ token_seq,
                                                                 const int* __restrict__ token_pos, int kw, int vw,
                                                                 int block_size, int max_blocks) {
  const int64_t t = blockIdx.x;
  const int seq = token_seq[t], pos = token_pos[t];
  const int64_t row = (int64_t)block_tables[(int64_t)seq * max_blocks + pos / block_size] * block_size + pos % block_size;
  for (int i = threadIdx.x; i < kw; i += blockDim.x) k_cache[row * kw + i] = k[t * ldk + i];
  for (int i = threadIdx.x; i < vw; i += blockDim.x) {
    T val = v[t * ldv + i];
    if (v_other != nullptr)
      val = from_f32<T>((1.f - lam) * to_f32<T>(val) + lam * to_f32<T>(v_other[t * ldvo + i]));
    v_cache[row * vw + i] = val;
  }
}

// ------------------------------------------------------------------------------------------------ paged attention
// One warp per (step token, query head).  Keys 0..pos of the token's sequence are walked in tiles of 32 in a fixed order
// (lane = key for the scores, lane = value channel for the weighted sum), online softmax in fp32.  With `sink` the running
// maximum starts at 0 and the denominator at 1: a key of score 0 without a value.
constexpr int ATT_MAX_VREG = 8;   // value width up to 256

template <typename T>
__global__ void __launch_bounds__(128) paged_bias_attention_kernel(
    const T* __restrict__ q, int64_t ldq, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
    const int* __restrict__ block_tables, const int* __restrict__ token_seq, const int* __restrict__ token_pos,
    const float* __restrict__ bias_table, const int* __restrict__ bucket_start, int nbuckets, T* __restrict__ out,
    int64_t tokens, int heads, int kv_heads, int dim, int vdim, int block_size, int max_blocks, float scale, int sink) {
  extern __shared__ float smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  float* qs = smem + warp * dim;
  int* bstart = reinterpret_cast<int*>(smem + nwarps * dim);
  for (int i = threadIdx.x; i < nbuckets; i += blockDim.x) bstart[i] = bucket_start[i];
  const int64_t unit = (int64_t)blockIdx.x * nwarps + warp;
  const bool live = unit < tokens * heads;
  const int64_t t = live ? unit / heads : 0;
  const int h = live ? (int)(unit % heads) : 0;
  for (int i = lane; i < dim; i += 32) qs[i] = live ? to_f32<T>(q[t * ldq + h * dim + i]) * scale : 0.f;
  __syncthreads();
  if (!live) return;
  const int g = h / (heads / kv_heads);
  const int seq = token_seq[t], pos = token_pos[t];
  const int* bt = block_tables + (int64_t)seq * max_blocks;
  const int half = nbuckets >> 1;
  float m = sink ? 0.f : -INFINITY, l = sink ? 1.f : 0.f;
  float acc[ATT_MAX_VREG];
#pragma unroll
  for (int r = 0; r < ATT_MAX_VREG; ++r) acc[r] = 0.f;
  for (int j0 = 0; j0 <= pos; j0 += 32) {
    const int jk = j0 + lane;
    float sc = -INFINITY;
    int64_t myrow = 0;
    if (jk <= pos) {
      myrow = ((int64_t)bt[jk / block_size] * block_size + jk % block_size) * kv_heads + g;
      const T* kr = k_cache + myrow * dim;
      float d0 = 0.f, d1 = 0.f;
      int i = 0;
      for (; i + 1 < dim; i += 2) {
        d0 = fmaf(qs[i], to_f32<T>(kr[i]), d0);
        d1 = fmaf(qs[i + 1], to_f32<T>(kr[i + 1]), d1);
      }
      if (i < dim) d0 = fmaf(qs[i], to_f32<T>(kr[i]), d0);
      sc = d0 + d1;
      if (nbuckets > 0) {
        const int n = pos - jk;
        int b = n;
        if (n >= half) {
          b = half;
          while (b + 1 < nbuckets && bstart[b + 1] <= n) ++b;
        }
        sc += bias_table[b * heads + h];
      }
    }
    const float mn = fmaxf(m, warp_max(sc));
    const float alpha = expf(m - mn);           // m = -inf only before the first tile without a sink: exp(-inf) = 0
    const float pj = jk <= pos ? expf(sc - mn) : 0.f;
    l = l * alpha + warp_sum(pj);
    m = mn;
#pragma unroll
    for (int r = 0; r < ATT_MAX_VREG; ++r) acc[r] *= alpha;
    const int nk = min(32, pos - j0 + 1);
    for (int jj = 0; jj < nk; ++jj) {
      const float pw = __shfl_sync(0xffffffffu, pj, jj);
      const int64_t vrow = __shfl_sync(0xffffffffu, myrow, jj);
      const T* vr = v_cache + vrow * vdim;
#pragma unroll
      for (int r = 0; r < ATT_MAX_VREG; ++r) {
        const int c = lane + 32 * r;
        if (c < vdim) acc[r] = fmaf(pw, to_f32<T>(vr[c]), acc[r]);
      }
    }
  }
  const float inv = 1.f / l;
#pragma unroll
  for (int r = 0; r < ATT_MAX_VREG; ++r) {
    const int c = lane + 32 * r;
    if (c < vdim) out[t * ((int64_t)heads * vdim) + h * vdim + c] = from_f32<T>(acc[r] * inv);
  }
}

// ------------------------------------------------------------------------------------------------ tensor-core variant
// 16-bit inputs: a CTA of 4 warps owns 64 query ROWS of one (sequence, kv head): row = (token of the portion, query head
// of the kv head's group), so the K / V tile that cp.async brings from the pages is shared by the whole group and a
// decoded token fills rows with its group's heads.  S = Q K^T and O += P V run on mma.sync m16n8k16 with fp32
// accumulators; softmax, bias and sink in fp32 registers.  D = head width rounded up (zero padded in shared memory).
constexpr int MMA_BM = 64, MMA_BN = 64;

template <typename T> CB_DEVICE void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <> CB_DEVICE void mma_16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <> CB_DEVICE void mma_16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T> CB_DEVICE uint32_t pack2(float lo, float hi);
template <> CB_DEVICE uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> CB_DEVICE uint32_t pack2<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
CB_DEVICE float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
CB_DEVICE void cp_async16(void* smem_dst, const void* gmem_src, uint32_t src_bytes) {
  const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem_src), "r"(src_bytes) : "memory");
}

template <typename T, int D>
__global__ void __launch_bounds__(128) paged_bias_attention_mma_kernel(
    const T* __restrict__ q, int64_t ldq, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
    const int* __restrict__ block_tables, const int* __restrict__ cu_q, const int* __restrict__ ctx_len,
    const float* __restrict__ bias_table, const uint8_t* __restrict__ lut, int lut_n, int nbuckets, T* __restrict__ out,
    int heads, int kv_heads, int dim, int vdim, int block_size, int max_blocks, float scale, int sink) {
  constexpr int LDS = D + 8;                    // padded row: 16-byte aligned, conflict-free fragment reads
  constexpr float LOG2E = 1.4426950408889634f;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* Ks = reinterpret_cast<T*>(smem_raw);
  T* Vs = Ks + MMA_BN * LDS;
  float* tab = reinterpret_cast<float*>(Vs + MMA_BN * LDS);          // [nbuckets][R] of this kv head's group
  const int s = blockIdx.z, g = blockIdx.y;
  const int R = heads / kv_heads;
  const int t0 = cu_q[s], qlen = cu_q[s + 1] - t0;
  const int nrows = qlen * R, row0 = blockIdx.x * MMA_BM;
  if (row0 >= nrows) return;
  const int ctx = ctx_len[s];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gid = lane >> 2, tig = lane & 3;
  for (int i = tid; i < nbuckets * R; i += blockDim.x) tab[i] = bias_table[(i / R) * heads + g * R + (i % R)] * LOG2E;
  const int* bt = block_tables + (int64_t)s * max_blocks;

  int rr[2], pos[2], hr[2];
  bool valid[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    rr[e] = row0 + warp * 16 + gid + 8 * e;
    valid[e] = rr[e] < nrows;
    hr[e] = valid[e] ? rr[e] % R : 0;
    pos[e] = valid[e] ? ctx + rr[e] / R : -1;
  }
  uint32_t qf[D / 16][4];
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = e & 1, col = ks * 16 + tig * 2 + ((e >> 1) ? 8 : 0);
      uint32_t val = 0;
      if (valid[r] && col < dim)
        val = *reinterpret_cast<const uint32_t*>(q + (int64_t)(t0 + rr[r] / R) * ldq + (g * R + hr[r]) * dim + col);
      qf[ks][e] = val;
    }
  float o[D / 8][4];
#pragma unroll
  for (int nv = 0; nv < D / 8; ++nv)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[nv][e] = 0.f;
  float m[2], l[2];
  m[0] = m[1] = sink ? 0.f : -INFINITY;         // log2 domain (0 either way)
  l[0] = l[1] = 0.f;                            // per-thread partial; the sink's 1 is added once at the end
  const float sc2 = scale * LOG2E;
  const int last_row = min(nrows - 1, row0 + MMA_BM - 1);
  const int pos_max = ctx + last_row / R;

  for (int j0 = 0; j0 <= pos_max; j0 += MMA_BN) {
    __syncthreads();                            // previous tile fully consumed (and `tab` visible on the first pass)
    constexpr int CH = D / 8;
    for (int idx = tid; idx < MMA_BN * CH; idx += blockDim.x) {
      const int r = idx / CH, c8 = (idx % CH) * 8;
      const int j = j0 + r;
      const bool in = j <= pos_max;
      const int64_t row = in ? ((int64_t)bt[j / block_size] * block_size + j % block_size) * kv_heads + g : 0;
      const bool kin = in && c8 < dim, vin = in && c8 < vdim;
      cp_async16(Ks + r * LDS + c8, k_cache + (kin ? row * dim + c8 : 0), kin ? 16u : 0u);
      cp_async16(Vs + r * LDS + c8, v_cache + (vin ? row * vdim + c8 : 0), vin ? 16u : 0u);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    const int wmax = ctx + min(nrows - 1, row0 + warp * 16 + 15) / R;     // last position any row of this warp sees
    if (j0 > wmax) continue;                                              // warp-uniform: whole tile masked
    float sacc[MMA_BN / 8][4];
#pragma unroll
    for (int nt = 0; nt < MMA_BN / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) sacc[nt][e] = 0.f;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const T* kp = Ks + (nt * 8 + gid) * LDS + ks * 16 + tig * 2;
        mma_16816<T>(sacc[nt], qf[ks], *reinterpret_cast<const uint32_t*>(kp), *reinterpret_cast<const uint32_t*>(kp + 8));
      }
    }
    float mx[2] = {m[0], m[1]};
#pragma unroll
    for (int nt = 0; nt < MMA_BN / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1, j = j0 + nt * 8 + tig * 2 + (e & 1);
        float sv = -INFINITY;
        if (j <= pos[r]) {
          sv = sacc[nt][e] * sc2;
          if (nbuckets > 0) {
            const int n = pos[r] - j;
            const int b = n < lut_n ? (int)__ldg(lut + n) : nbuckets - 1;
            sv += tab[b * R + hr[r]];
          }
        }
        sacc[nt][e] = sv;
        mx[r] = fmaxf(mx[r], sv);
      }
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float mu = mx[r] == -INFINITY ? 0.f : mx[r];
      alpha[r] = ex2f(m[r] - mu);                 // m = -inf -> 0
      m[r] = mx[r];
      l[r] *= alpha[r];
      mx[r] = mu;
    }
#pragma unroll
    for (int nv = 0; nv < D / 8; ++nv) {
      o[nv][0] *= alpha[0]; o[nv][1] *= alpha[0];
      o[nv][2] *= alpha[1]; o[nv][3] *= alpha[1];
    }
#pragma unroll
    for (int nt = 0; nt < MMA_BN / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p = ex2f(sacc[nt][e] - mx[e >> 1]);
        sacc[nt][e] = p;
        l[e >> 1] += p;
      }
#pragma unroll
    for (int kk = 0; kk < MMA_BN / 16; ++kk) {
      uint32_t pa[4];
      pa[0] = pack2<T>(sacc[2 * kk][0], sacc[2 * kk][1]);
      pa[1] = pack2<T>(sacc[2 * kk][2], sacc[2 * kk][3]);
      pa[2] = pack2<T>(sacc[2 * kk + 1][0], sacc[2 * kk + 1][1]);
      pa[3] = pack2<T>(sacc[2 * kk + 1][2], sacc[2 * kk + 1][3]);
      const uint32_t vrow = (uint32_t)__cvta_generic_to_shared(Vs + (kk * 16 + (lane & 15)) * LDS);
#pragma unroll
      for (int nv = 0; nv < D / 8; ++nv) {
        uint32_t b0, b1;
        asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];"
                     : "=r"(b0), "=r"(b1) : "r"(vrow + nv * 16));
        mma_16816<T>(o[nv], pa, b0, b1);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    if (sink) l[r] += ex2f(0.f - (m[r] == -INFINITY ? 0.f : m[r]));
    if (!valid[r]) continue;
    const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
    T* orow = out + (int64_t)(t0 + rr[r] / R) * ((int64_t)heads * vdim) + (g * R + hr[r]) * vdim;
#pragma unroll
    for (int nv = 0; nv < D / 8; ++nv) {
      const int c = nv * 8 + tig * 2;
      if (c < vdim) *reinterpret_cast<uint32_t*>(orow + c) = pack2<T>(o[nv][2 * r] * inv, o[nv][2 * r + 1] * inv);
    }
  }
}

template <typename T, int D>
int launch_attention_mma(const void* q, int64_t ldq, const void* k_cache, const void* v_cache, const int* block_tables,
                         const int* cu_q, const int* ctx_len, const float* bias_table, const uint8_t* lut, int lut_n,
                         int nbuckets, void* out, int nseq, int max_q, int heads, int kv_heads, int dim, int vdim,
                         int block_size, int max_blocks, float scale, int sink, cudaStream_t st) {
  const int R = heads / kv_heads;
  const size_t smem = (size_t)2 * MMA_BN * (D + 8) * sizeof(T) + (size_t)nbuckets * R * sizeof(float);
  auto kern = paged_bias_attention_mma_kernel<T, D>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  dim3 grid((max_q * R + MMA_BM - 1) / MMA_BM, kv_heads, nseq);
  kern<<<grid, 128, smem, st>>>((const T*)q, ldq, (const T*)k_cache, (const T*)v_cache, block_tables, cu_q, ctx_len,
                                bias_table, lut, lut_n, nbuckets, (T*)out, heads, kv_heads, dim, vdim, block_size,
                                max_blocks, scale, sink);
  return CB_LAUNCH_CHECK();
}

}  // namespace

// ================================================================================================ C launchers
extern "C" {

int cb_short_conv_silu(const void* x, int64_t ldx, const void* w, void* state, void* out, int64_t ldo, const int* cu_q,
                       const int* ctx_len, const int* slots, int nseq, int max_q, int C, int taps, int apply_silu,
                       int update_state, int dtype, cudaStream_t st) {
  if (taps < 1 || taps > CONV_MAX_TAPS) return (int)cudaErrorInvalidValue;
  if (nseq == 0 || max_q == 0) return 0;
  dim3 grid((C + 127) / 128, (max_q + CONV_TOK_TILE - 1) / CONV_TOK_TILE, nseq);
  CB_DISPATCH_FLOAT(dtype, T, {
    short_conv_silu_kernel<T><<<grid, 128, 0, st>>>((const T*)x, ldx, (const T*)w, (const T*)state, (T*)out, ldo, cu_q,
                                                    ctx_len, slots, C, taps, apply_silu);
    if (update_state && taps > 1)
      short_conv_state_kernel<T><<<dim3((C + 127) / 128, nseq), 128, 0, st>>>((const T*)x, ldx, (T*)state, cu_q, ctx_len,
                                                                             slots, C, taps);
  });
  return CB_LAUNCH_CHECK();
}

int cb_state_scan(int mode, const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv,
                  const void* araw, int64_t lda, const void* braw, int64_t ldb, const float* head_decay,
                  const float* a_log, const float* dt_bias, float* state, float* out, const int* cu_q,
                  const int* ctx_len, const int* slots, int nseq, int heads, int qk_heads, int dim, int vdim,
                  int act_silu, int unit_qk, float unit_eps, float q_scale, int dtype, cudaStream_t st) {
  if (nseq == 0) return 0;
  if (heads % qk_heads != 0) return (int)cudaErrorInvalidValue;
  ScanParams p{q, k, v, ldq, ldk, ldv, araw, lda, braw, ldb, head_decay, a_log, dt_bias, state, out, cu_q, ctx_len, slots,
               heads, qk_heads, dim, vdim, act_silu, unit_qk, unit_eps, q_scale};
  CB_DISPATCH_FLOAT(dtype, T, {
    if (mode == SCAN_DELTA) return launch_scan<SCAN_DELTA, T>(p, nseq, st);
    return launch_scan<SCAN_DECAY, T>(p, nseq, st);
  });
  return CB_LAUNCH_CHECK();
}

int cb_gated_group_rmsnorm(const float* o, const void* w, int wn, const void* gate, int64_t ldg, void* out, int64_t tokens,
                           int C, int group, float eps, int dtype, cudaStream_t st) {
  if (tokens == 0) return 0;
  if (group <= 0 || C % group != 0) return (int)cudaErrorInvalidValue;
  const int64_t units = tokens * (C / group);
  CB_DISPATCH_FLOAT(dtype, T, {
    gated_group_rmsnorm_kernel<T><<<(unsigned)((units + 7) / 8), 256, 0, st>>>(o, (const T*)w, wn, (const T*)gate, ldg,
                                                                              (T*)out, tokens, C, group, eps);
  });
  return CB_LAUNCH_CHECK();
}

int cb_rmsnorm_residual(float* x, const void* y, int64_t ldy, const void* w, void* h, int64_t tokens, int W, float eps,
                        float mult, float offset, int dtype, cudaStream_t st) {
  if (tokens == 0) return 0;
  CB_DISPATCH_FLOAT(dtype, T, {
    rmsnorm_residual_kernel<T><<<(unsigned)tokens, 256, 0, st>>>(x, (const T*)y, ldy, (const T*)w, (T*)h, W, eps, mult,
                                                                offset);
  });
  return CB_LAUNCH_CHECK();
}

int cb_rmsnorm_f32in(const float* x, const void* w, void* out, int64_t tokens, int W, float eps, float offset, int dtype,
                     cudaStream_t st) {
  if (tokens == 0) return 0;
  CB_DISPATCH_FLOAT(dtype, T, {
    rmsnorm_f32in_kernel<T><<<(unsigned)tokens, 256, 0, st>>>(x, (const T*)w, (T*)out, W, eps, offset);
  });
  return CB_LAUNCH_CHECK();
}

int cb_paged_kv_write_mix(const void* k, int64_t ldk, const void* v, int64_t ldv, const void* v_other, int64_t ldvo,
                          float lam, void* k_cache, void* v_cache, const int* block_tables, const int* token_seq,
                          const int* token_pos, int64_t tokens, int kw, int vw, int block_size, int max_blocks, int dtype,
                          cudaStream_t st) {
  if (tokens == 0) return 0;
  CB_DISPATCH_FLOAT(dtype, T, {
    paged_kv_write_mix_kernel<T><<<(unsigned)tokens, 128, 0, st>>>((const T*)k, ldk, (const T*)v, ldv, (const T*)v_other,
                                                                  ldvo, lam, (T*)k_cache, (T*)v_cache, block_tables,
                                                                  token_seq, token_pos, kw, vw, block_size, max_blocks);
  });
  return CB_LAUNCH_CHECK();
}

int cb_paged_bias_attention(const void* q, int64_t ldq, const void* k_cache, const void* v_cache, const int* block_tables,
                            const int* token_seq, const int* token_pos, const float* bias_table, const int* bucket_start,
                            int nbuckets, void* out, int64_t tokens, int heads, int kv_heads, int dim, int vdim,
                            int block_size, int max_blocks, float scale, int sink, int dtype, cudaStream_t st) {
  if (tokens == 0) return 0;
  if (vdim > 32 * ATT_MAX_VREG || heads % kv_heads != 0) return (int)cudaErrorInvalidValue;
  const int nwarps = 4;
  const size_t smem = (size_t)nwarps * dim * sizeof(float) + (size_t)nbuckets * sizeof(int);
  const int64_t units = tokens * heads;
  CB_DISPATCH_FLOAT(dtype, T, {
    paged_bias_attention_kernel<T><<<(unsigned)((units + nwarps - 1) / nwarps), nwarps * 32, smem, st>>>(
        (const T*)q, ldq, (const T*)k_cache, (const T*)v_cache, block_tables, token_seq, token_pos, bias_table,
        bucket_start, nbuckets, (T*)out, tokens, heads, kv_heads, dim, vdim, block_size, max_blocks, scale, sink);
  });
  return CB_LAUNCH_CHECK();
}

// 16-bit dtypes, widths that are multiples of 8 and at most 128: the tensor-core kernel
int cb_paged_bias_attention_mma(const void* q, int64_t ldq, const void* k_cache, const void* v_cache,
                                const int* block_tables, const int* cu_q, const int* ctx_len, const float* bias_table,
                                const uint8_t* lut, int lut_n, int nbuckets, void* out, int nseq, int max_q, int heads,
                                int kv_heads, int dim, int vdim, int block_size, int max_blocks, float scale, int sink,
                                int dtype, cudaStream_t st) {
  if (nseq == 0 || max_q == 0) return 0;
  if (heads % kv_heads != 0 || dim % 8 != 0 || vdim % 8 != 0 || dim > 128 || vdim > 128 || (ldq & 1))
    return (int)cudaErrorInvalidValue;
  const int dmax = dim > vdim ? dim : vdim;
#define CB_ATT_MMA(T, D)                                                                                              \
  return launch_attention_mma<T, D>(q, ldq, k_cache, v_cache, block_tables, cu_q, ctx_len, bias_table, lut, lut_n,   \
                                    nbuckets, out, nseq, max_q, heads, kv_heads, dim, vdim, block_size, max_blocks,  \
                                    scale, sink, st)
  CB_DISPATCH_HALF(dtype, T, {
    if (dmax <= 32) { CB_ATT_MMA(T, 32); }
    else if (dmax <= 64) { CB_ATT_MMA(T, 64); }
    else { CB_ATT_MMA(T, 128); }
  });
#undef CB_ATT_MMA
  return CB_LAUNCH_CHECK();
}

}  // extern "C"
