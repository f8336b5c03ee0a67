// seq_mixers.cu — ragged-batch kernels for layer stacks that mix attention with recurrent sequence mixers
// (gated delta rule, state-space duality) and keep the residual stream in fp32.
//
// Every kernel works on a ragged batch: `tok_seq[t]` / `tok_pos[t]` give each token's sequence slot in the batch and
// its position in its sequence, `seq_info[s] = {first row, rows, tokens already seen, state slot}` describes each
// sequence, `block_tables[s]` its pages of the key/value cache.  `T` is the activation type (bf16 when serving,
// float for exact evaluation); everything that the recurrences, norms and softmax touch is fp32 in both.
//
//   embed_sinusoid        token row * scale (+ sinusoidal position vector)          -> fp32 residual
//   resid_norm_step       residual += rms(y) * w_post (+ extra);  out = rms(residual) * w_pre   (one pass per row)
//   qk_norm_append        bias + per-head unit-RMS of q and k, q -> fp32, k / v -> paged cache
//   sink_attention        causal, chunk-local or sliding-window softmax attention over the paged cache with a per-head
//                         sink logit; values may be a column range of the key rows (attention in a latent space)
//   conv_silu / conv_state_update   short causal per-channel filter with its carried inputs per state slot
//   unit_norm_heads, recurrence_gates   per-head L2 normalisation; decay / write strength of the recurrences
//   linear_recurrence     S <- a S;  u = b (v - [delta] S^T k);  S <- S + k u^T;  o = S^T q (+ D v), state per slot
//   group_norm_gate       RMS norm over channel groups combined with a SiLU gate (before or after the norm)
//   gated_act_rows, bias_act_rows   act(gate) * up, act(x + bias) for any width and fp32 or bf16 rows
//   conv_residual, post_norm_mix, rms_scale_rows   post-norm layers: x + filter(x) in front of a sublayer,
//                         x += scale (.) rms(y) * gain behind it (+ a weighted sum of all layers' streams), final norm
//   rms_norm_slice, latent_qk_prepare   latent attention: query latent norm; key latent norm + rotation + cache append
//   mlstm_prepare / mlstm_gate_scan / mlstm_output   matrix-memory LSTM around linear_recurrence
//   channel_decay_gates   decay per (head, key channel) pair for linear_recurrence (its per-channel form), sigmoid write strength
//   sigmoid_gate_rows, power_norm_act   sigmoid gate per channel or per head in place; p1 z/rms(z) + p2 z^2/rms(z^2) + p3 z^3/rms(z^3) + p0
#include <algorithm>
#include "sxb_common.cuh"
#include <cuda_pipeline.h>

namespace sxb {
namespace seqmix {



#define SEQMIX_DISPATCH(dtype, ...)                \
  do {                                             \
    if ((dtype) == 0) {                         \
      using T = float;                             \
      __VA_ARGS__;                                 \
    } else if ((dtype) == 2) {                 \
      using T = __nv_bfloat16;                     \
      __VA_ARGS__;                                 \
    } else {                                       \
      return SXB_ERR_UNSUPPORTED;                  \
    }                                              \
  } while (0)

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 30.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

// ------------------------------------------------------------------------------------------------ embedding
template <typename T>
__global__ void __launch_bounds__(256)
embed_sinusoid_kernel(const int* __restrict__ ids, const int* __restrict__ pos, const T* __restrict__ table,
                      float* __restrict__ out, int width, float scale, float base) {
  const int t = blockIdx.x;
  const T* row = table + (long long)ids[t] * width;
  const float p = (float)pos[t];
  const float lb = log2f(base);
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const int i = c >> 1;
    const float freq = exp2f(-(2.f * (float)i / (float)width) * lb);
    const float ang = p * freq;
    const float pe = base > 0.f ? ((c & 1) ? cosf(ang) : sinf(ang)) : 0.f;      // base <= 0: no position vector
    out[(long long)t * width + c] = to_f32<T>(row[c]) * scale + pe;
  }
}

// ------------------------------------------------------------------------------------------------ residual + norms
// One CTA per row.  y (optional): residual += mult * y / rms(y) * w_post, or += mult * y without w_post; with y_scale
// the addend is also multiplied per channel by y_scale.  extra (optional): residual += extra.  w_pre (optional):
// out = residual / rms(residual) * (w_add + w_pre) (w_add 1 for weights stored as their distance from one); out without
// w_pre: the residual itself in the activation type.
template <typename T>
__global__ void __launch_bounds__(256)
resid_norm_step_kernel(float* __restrict__ resid, const T* __restrict__ y, const T* __restrict__ w_post,
                       const float* __restrict__ extra, const T* __restrict__ w_pre, T* __restrict__ out, int width,
                       float eps, float mult, const T* __restrict__ y_scale, float w_add) {
  __shared__ float red[32];
  const long long base = (long long)blockIdx.x * width;
  float* r = resid + base;
  float inv_y = mult;
  if (y != nullptr && w_post != nullptr) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
      const float v = to_f32<T>(y[base + c]);
      ss += v * v;
    }
    ss = block_sum(ss, red);
    inv_y = mult / sqrtf(ss / (float)width + eps);
  }
  float ss2 = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = r[c];
    if (y != nullptr) {
      float add = to_f32<T>(y[base + c]) * inv_y * (w_post ? to_f32<T>(w_post[c]) : 1.f);
      if (y_scale != nullptr) add *= to_f32<T>(y_scale[c]);
      v += add;
    }
    if (extra != nullptr) v += extra[base + c];
    if (y != nullptr || extra != nullptr) r[c] = v;
    ss2 += v * v;
  }
  if (out == nullptr) return;
  if (w_pre == nullptr) {
    for (int c = threadIdx.x; c < width; c += blockDim.x) out[base + c] = from_f32<T>(r[c]);
    return;
  }
  ss2 = block_sum(ss2, red);
  const float inv = 1.f / sqrtf(ss2 / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    out[base + c] = from_f32<T>(r[c] * inv * (w_add + to_f32<T>(w_pre[c])));
}

// ------------------------------------------------------------------------------------------------ attention
// One CTA per token, one warp per head slot (Hq query heads, G key heads, G value heads in the fused projection row).
template <typename T>
__global__ void __launch_bounds__(128)
qk_norm_append_kernel(const T* __restrict__ qkv, long long ld, const T* __restrict__ bias, float* __restrict__ q_out,
                      T* __restrict__ kcache, T* __restrict__ vcache, const int* __restrict__ tok_seq,
                      const int* __restrict__ tok_pos, const int* __restrict__ tables, int max_blocks, int block_size,
                      int Hq, int G, int d, int dv, float eps, int normalize) {
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const T* row = qkv + (long long)t * ld;
  const int pos = tok_pos[t];
  const long long page = tables[(long long)tok_seq[t] * max_blocks + pos / block_size];
  const long long slot = page * block_size + pos % block_size;
  for (int s = warp; s < Hq + 2 * G; s += nw) {
    if (s < Hq + G) {
      const int col = s * d;     // q heads then k heads are contiguous with the same head size
      float ss = 0.f;
      for (int c = lane; c < d; c += 32) {
        const float v = to_f32<T>(row[col + c]) + (bias ? to_f32<T>(bias[col + c]) : 0.f);
        ss += v * v;
      }
      ss = warp_sum(ss);
      const float inv = normalize ? 1.f / sqrtf(ss / (float)d + eps) : 1.f;
      for (int c = lane; c < d; c += 32) {
        const float v = (to_f32<T>(row[col + c]) + (bias ? to_f32<T>(bias[col + c]) : 0.f)) * inv;
        if (s < Hq) q_out[((long long)t * Hq + s) * d + c] = v;
        else kcache[(slot * G + (s - Hq)) * d + c] = from_f32<T>(v);
      }
    } else {
      const int g = s - Hq - G, col = (Hq + G) * d + g * dv;
      for (int c = lane; c < dv; c += 32) {
        const float v = to_f32<T>(row[col + c]) + (bias ? to_f32<T>(bias[col + c]) : 0.f);
        vcache[(slot * G + g) * dv + c] = from_f32<T>(v);
      }
    }
  }
}

// The same append for projections that pass a short causal filter first.  One warp per (token, head slot): grid
// (tokens, ceil(slots / 4)), four warps per CTA.  A lane holds VEC consecutive channels of its head (VEC = head size / 32
// rounded up to a power of two, head sizes up to 256) and moves them with one access of VEC elements when the head sizes
// and the row pitch allow.  Every channel of q | k | v is filtered over time (w [C, taps], last tap = current token;
// earlier inputs from this batch's rows, else from the slot's carried inputs state [slots, taps-1, C], else zero; w null:
// no filter), q and k heads are divided by their root mean square and multiplied by a weight of d entries that all
// heads share (null: none), and q by 1 + coef * ln(floor((pos + 1) / every) + 1).  Filter sums, norms and the
// temperature are fp32.
template <typename T, int VEC>
struct alignas(sizeof(T) * VEC) Pack {
  T v[VEC];
};

template <typename T, int VEC>
__device__ __forceinline__ void load_pack(const T* p, float* o, bool vec, int valid) {
  if (vec) {
    const Pack<T, VEC> pk = *reinterpret_cast<const Pack<T, VEC>*>(p);
#pragma unroll
    for (int i = 0; i < VEC; ++i) o[i] = to_f32<T>(pk.v[i]);
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) o[i] = i < valid ? to_f32<T>(p[i]) : 0.f;
  }
}

template <typename T, int VEC>
__device__ __forceinline__ void store_pack(T* p, const float* o, bool vec, int valid) {
  if (vec) {
    Pack<T, VEC> pk;
#pragma unroll
    for (int i = 0; i < VEC; ++i) pk.v[i] = from_f32<T>(o[i]);
    *reinterpret_cast<Pack<T, VEC>*>(p) = pk;
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i)
      if (i < valid) p[i] = from_f32<T>(o[i]);
  }
}

// TAPS > 0 (filters of 2 to 4 taps): a warp walks `rows_per_warp` consecutive batch rows with the filter's weights and
// the last TAPS-1 inputs in registers; the inputs are fetched by the rule above at the warp's first row and at a
// sequence's first row in the batch, and shifted otherwise.  TAPS == 0: any number of taps (or none), one row per warp.
template <typename T, int VEC, int TAPS>
__global__ void __launch_bounds__(128)
qkv_filter_norm_append_kernel(const T* __restrict__ qkv, long long ld, const T* __restrict__ w,
                              const T* __restrict__ state, const int* __restrict__ seq_info,
                              const T* __restrict__ q_w, const T* __restrict__ k_w, float* __restrict__ q_out,
                              T* __restrict__ kcache, T* __restrict__ vcache, const int* __restrict__ tok_seq,
                              const int* __restrict__ tok_pos, const int* __restrict__ tables, int max_blocks,
                              int block_size, int Hq, int G, int d, int dv, int taps, float eps, int normalize,
                              float temp_coef, int temp_every, int vec_ok, int n_tokens, int rows_per_warp) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int s = blockIdx.y * 4 + warp;
  if (s >= Hq + 2 * G) return;
  const int C = (Hq + G) * d + G * dv;
  const bool is_v = s >= Hq + G;
  const int n = is_v ? dv : d;
  const int col = is_v ? (Hq + G) * d + (s - Hq - G) * dv : s * d;
  const int c0 = lane * VEC;
  const int valid = min(VEC, n - c0);          // channels of this lane (<= 0: none)
  const bool vec = vec_ok && valid == VEC;
  const int ch = col + c0;
  const T* hw = is_v ? nullptr : (s < Hq ? q_w : k_w);
  float gain[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) gain[i] = (hw && i < valid) ? to_f32<T>(hw[c0 + i]) : 1.f;
  constexpr int NT = TAPS > 0 ? TAPS : 1;
  float wt[VEC][NT], hist[NT][VEC];
  if (TAPS > 0) {
#pragma unroll
    for (int i = 0; i < VEC; ++i)
#pragma unroll
      for (int j = 0; j < NT; ++j) wt[i][j] = i < valid ? to_f32<T>(w[(long long)(ch + i) * NT + j]) : 0.f;
  }
  const int t0 = blockIdx.x * rows_per_warp, t1 = min(t0 + rows_per_warp, n_tokens);
  for (int t = t0; t < t1; ++t) {
    const int pos = tok_pos[t];
    const int* si = seq_info + 4 * tok_seq[t];
    const int local = t - si[0], seen = si[2];
    const T* st = state ? state + (long long)si[3] * (taps - 1) * C : nullptr;
    float v[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) v[i] = 0.f;
    if (valid > 0) {
      if (TAPS > 0) {
        if (t == t0 || local == 0) {
#pragma unroll
          for (int j = 1; j < NT; ++j) {
            const int src = local - j;
            if (src >= 0) load_pack<T, VEC>(qkv + (long long)(t - j) * ld + ch, hist[j], vec, valid);
            else if (seen + src >= 0) load_pack<T, VEC>(st + (long long)(NT - 1 + src) * C + ch, hist[j], vec, valid);
            else {
#pragma unroll
              for (int i = 0; i < VEC; ++i) hist[j][i] = 0.f;
            }
          }
        } else {
#pragma unroll
          for (int j = NT - 1; j >= 1; --j)
#pragma unroll
            for (int i = 0; i < VEC; ++i) hist[j][i] = hist[j - 1][i];
        }
        load_pack<T, VEC>(qkv + (long long)t * ld + ch, hist[0], vec, valid);
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
          for (int i = 0; i < VEC; ++i) v[i] += wt[i][NT - 1 - j] * hist[j][i];
      } else if (w == nullptr) {
        load_pack<T, VEC>(qkv + (long long)t * ld + ch, v, vec, valid);
      } else {
        for (int j = 0; j < taps; ++j) {
          const int src = local - j;
          float u[VEC];
          if (src >= 0) load_pack<T, VEC>(qkv + (long long)(t - j) * ld + ch, u, vec, valid);
          else if (seen + src >= 0) load_pack<T, VEC>(st + (long long)(taps - 1 + src) * C + ch, u, vec, valid);
          else continue;
#pragma unroll
          for (int i = 0; i < VEC; ++i)
            if (i < valid) v[i] += to_f32<T>(w[(long long)(ch + i) * taps + (taps - 1 - j)]) * u[i];
        }
      }
    }
    float inv = 1.f;
    if (!is_v) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < VEC; ++i) ss += v[i] * v[i];
      ss = warp_sum(ss);
      if (normalize) inv = 1.f / sqrtf(ss / (float)d + eps);
      if (s < Hq && temp_coef != 0.f) inv *= 1.f + temp_coef * logf((float)((pos + 1) / temp_every + 1));
    }
    if (valid <= 0) continue;
    float o[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) o[i] = v[i] * inv * gain[i];
    if (s < Hq) {
      store_pack<float, VEC>(q_out + ((long long)t * Hq + s) * d + c0, o, vec, valid);
    } else {
      const long long page = tables[(long long)tok_seq[t] * max_blocks + pos / block_size];
      const long long slot = page * block_size + pos % block_size;
      if (!is_v) store_pack<T, VEC>(kcache + (slot * G + (s - Hq)) * d + c0, o, vec, valid);
      else store_pack<T, VEC>(vcache + (slot * G + (s - Hq - G)) * dv + c0, o, vec, valid);
    }
  }
}

// First position a query at `pos` attends to: the start of its aligned chunk (chunk > 0), else the start of a sliding
// window of `window` positions that ends at the query (window > 0), else the start of the sequence.
__device__ __forceinline__ int first_key(int pos, int chunk, int window) {
  if (chunk > 0) return (pos / chunk) * chunk;
  return window > 0 ? max(0, pos - window + 1) : 0;
}

constexpr int kMaxVPerLane = 8;      // value head size <= 256
constexpr int kShortAtom = 16;       // atoms of at most this many queries run one warp per (query, head)
constexpr int kBQ = 64, kBK = 64;    // query rows / keys per tile of the tiled kernel

template <typename T>
__device__ __forceinline__ float4 load4_f32(const T* p);
template <>
__device__ __forceinline__ float4 load4_f32<float>(const float* p) {
  return *reinterpret_cast<const float4*>(p);
}
template <>
__device__ __forceinline__ float4 load4_f32<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}

// Tiled form for atoms of many queries (prompt portions): one CTA per (64 queries of an atom, query head).  Q (scaled),
// one 64-key tile of K and V (converted to fp32) and the tile's weights (in the key tile's place, once the scores are
// done: head sizes up to 128 then leave room for two CTAs per SM) sit in shared memory; 256 threads hold 4x4
// scores and 4 x (dv/16) outputs each.  Scores, online softmax with the sink logit, and the weighted sum are fp32 FMAs:
// the weights must stay 32-bit, so the products cannot go through the bf16 tensor path.
template <typename T, int NV>
__global__ void __launch_bounds__(256, NV <= 2 ? 2 : 1)
sink_attention_tile_kernel(const float* __restrict__ q, const T* __restrict__ kcache, const T* __restrict__ vcache,
                           const float* __restrict__ sink, T* __restrict__ out, const int* __restrict__ atoms,
                           const int* __restrict__ tables, int max_blocks, int block_size, int Hq, int G, int d,
                           int dv, float scale, int chunk, int window, int kpitch, int vpitch,
                           const float* __restrict__ dist_bias, int bias_len, const T* __restrict__ gate,
                           long long gate_ld) {
  extern __shared__ __align__(16) float smf[];
  const int dp = d + 4, vp = NV * 64, pp = kBK + 4;
  float* Qs = smf;
  float* Ks = Qs + kBQ * dp;
  float* Vs = Ks + max(kBK * dp, kBQ * pp);
  float* Ps = Ks;                    // the weights take the key tile's place once every warp has its scores
  const int* a = atoms + 6 * (blockIdx.x >> 1);
  const int sub = blockIdx.x & 1;
  const int nq = min(a[2] - sub * kBQ, kBQ);
  if (nq <= 0) return;
  const int row0 = a[1] + sub * kBQ, pos0 = a[3] + sub * kBQ;
  const int h = blockIdx.y, g = h / (Hq / G);
  const int* tab = tables + (long long)a[0] * max_blocks;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int d4 = d >> 2;
  for (int i = tid; i < kBQ * d4; i += 256) {
    const int r = i / d4, c = (i % d4) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < nq) v = *reinterpret_cast<const float4*>(q + ((long long)(row0 + r) * Hq + h) * d + c);
    v.x *= scale, v.y *= scale, v.z *= scale, v.w *= scale;
    *reinterpret_cast<float4*>(Qs + r * dp + c) = v;
  }
  // The products run as packed pairs (fma.f32x2: two 32-bit FMAs per lane and instruction), so scores and outputs are
  // held as float2.
  float m[4], l[4];
  float2 acc[4][NV * 2];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m[i] = sink ? sink[h] : -INFINITY;
    l[i] = sink ? 1.f : 0.f;
#pragma unroll
    for (int c = 0; c < NV * 2; ++c) acc[i][c] = make_float2(0.f, 0.f);
  }
  const int last = pos0 + nq - 1;
  const int kbeg = first_key(pos0, chunk, window);
  for (int k0 = kbeg; k0 <= last; k0 += kBK) {
    __syncthreads();
    for (int i = tid; i < kBK * d4; i += 256) {
      const int r = i / d4, c = (i % d4) * 4, kj = k0 + r;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (kj <= last) {
        const long long slot = (long long)tab[kj / block_size] * block_size + kj % block_size;
        v = load4_f32<T>(kcache + slot * kpitch + g * d + c);
      }
      *reinterpret_cast<float4*>(Ks + r * dp + c) = v;
    }
    for (int i = tid; i < kBK * (vp >> 2); i += 256) {
      const int r = i / (vp >> 2), c = (i % (vp >> 2)) * 4, kj = k0 + r;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (kj <= last && c < dv) {
        const long long slot = (long long)tab[kj / block_size] * block_size + kj % block_size;
        v = load4_f32<T>(vcache + slot * vpitch + g * dv + c);
      }
      *reinterpret_cast<float4*>(Vs + r * vp + c) = v;
    }
    __syncthreads();
    float2 s2[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s2[i][j] = make_float2(0.f, 0.f);
    for (int c = 0; c < d; c += 4) {
      float4 qv[4], kv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) qv[i] = *reinterpret_cast<const float4*>(Qs + (ty + 16 * i) * dp + c);
#pragma unroll
      for (int j = 0; j < 4; ++j) kv[j] = *reinterpret_cast<const float4*>(Ks + (tx + 16 * j) * dp + c);
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          s2[i][j] = __ffma2_rn(make_float2(qv[i].x, qv[i].y), make_float2(kv[j].x, kv[j].y), s2[i][j]);
          s2[i][j] = __ffma2_rn(make_float2(qv[i].z, qv[i].w), make_float2(kv[j].z, kv[j].w), s2[i][j]);
        }
    }
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = s2[i][j].x + s2[i][j].y;
    __syncthreads();       // every warp is done with the key tile: its space now holds the weights
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = ty + 16 * i, qp = pos0 + r;
      const int lo = first_key(qp, chunk, window);
      float mt = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int kj = k0 + tx + 16 * j;
        if (!(r < nq && kj <= qp && kj >= lo)) s[i][j] = -INFINITY;
        else if (dist_bias != nullptr) s[i][j] += __ldg(dist_bias + (long long)h * bias_len + min(qp - kj, bias_len - 1));
        mt = fmaxf(mt, s[i][j]);
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, o));
      const float mn = fmaxf(m[i], mt);
      const float corr = (mn == -INFINITY) ? 1.f : expf(m[i] - mn);
      float ps = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float p = (s[i][j] == -INFINITY) ? 0.f : expf(s[i][j] - mn);
        ps += p;
        Ps[r * pp + tx + 16 * j] = p;
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
      l[i] = l[i] * corr + ps;
      m[i] = mn;
#pragma unroll
      for (int c = 0; c < NV * 2; ++c) acc[i][c] = __fmul2_rn(acc[i][c], make_float2(corr, corr));
    }
    __syncwarp();          // a row of weights is written and read by the 16 threads of one half-warp
    for (int j = 0; j < kBK; j += 4) {
      float4 pv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) pv[i] = *reinterpret_cast<const float4*>(Ps + (ty + 16 * i) * pp + j);
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
#pragma unroll
        for (int n = 0; n < NV; ++n) {
          const float4 vv = *reinterpret_cast<const float4*>(Vs + (j + jj) * vp + n * 64 + tx * 4);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float p = jj == 0 ? pv[i].x : (jj == 1 ? pv[i].y : (jj == 2 ? pv[i].z : pv[i].w));
            const float2 p2 = make_float2(p, p);
            acc[i][n * 2] = __ffma2_rn(p2, make_float2(vv.x, vv.y), acc[i][n * 2]);
            acc[i][n * 2 + 1] = __ffma2_rn(p2, make_float2(vv.z, vv.w), acc[i][n * 2 + 1]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty + 16 * i;
    if (r >= nq) continue;
    const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
#pragma unroll
    for (int n = 0; n < NV; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int c = n * 64 + tx * 4 + e;
        const float2 a2 = acc[i][n * 2 + (e >> 1)];
        if (c < dv) {
          float o = ((e & 1) ? a2.y : a2.x) * inv;
          if (gate != nullptr) o *= sigmoid_f(to_f32<T>(gate[(long long)(row0 + r) * gate_ld + h * dv + c]));
          out[((long long)(row0 + r) * Hq + h) * dv + c] = from_f32<T>(o);
        }
      }
  }
}

// One CTA of kAW warps per (token, key/value head): single decode tokens and short portions.  Keys lo..pos of the token's
// sequence, lo = start of the token's chunk (chunk > 0) or 0; the warps take 32-key tiles in turn (a lane scores one
// key, whose row reaches it through a coalesced copy into shared memory; then the tile's weights are broadcast and the lanes hold the value channels) and
// their partial (max, sum, weighted values) are merged in shared memory.  The softmax denominator also holds
// exp(sink[h]): a logit without a key or a value.
template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const T* __restrict__ k, int d, bool vec) {
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  if (vec) {
    for (int c = 0; c < d; c += 8) {
      const float4 x = load4_f32<T>(k + c), y = load4_f32<T>(k + c + 4);
      a0 += q[c] * x.x + q[c + 4] * y.x;
      a1 += q[c + 1] * x.y + q[c + 5] * y.y;
      a2 += q[c + 2] * x.z + q[c + 6] * y.z;
      a3 += q[c + 3] * x.w + q[c + 7] * y.w;
    }
  } else {
    for (int c = 0; c < d; ++c) a0 += q[c] * to_f32<T>(k[c]);
  }
  return (a0 + a1) + (a2 + a3);
}

constexpr int kAW = 8;               // warps of the per-token attention kernel; they take the key tiles in turn
constexpr int kKeyLoads = 8;         // 16-byte key loads a lane issues before it stores the first one
constexpr int kValLoads = 8;         // value rows a warp has in flight

// REP query heads that share one key/value head are handled together: a loaded key or value row serves all of them.
// VPL: value channels a lane holds (4 for value heads up to 128, else 8).
template <typename T, int REP, int VPL>
__global__ void __launch_bounds__(32 * kAW)
sink_attention_kernel(const float* __restrict__ q, const T* __restrict__ kcache, const T* __restrict__ vcache,
                      const float* __restrict__ sink, T* __restrict__ out, const int* __restrict__ tok_seq,
                      const int* __restrict__ tok_pos, const int* __restrict__ tables, int max_blocks, int block_size,
                      int Hq, int G, int d, int dv, float scale, int chunk, int window, int kpitch, int vpitch,
                      const int* __restrict__ atoms, const float* __restrict__ dist_bias, int bias_len,
                      const T* __restrict__ gate, long long gate_ld) {
  // q [REP][d8] | partial values [kAW][REP][dv] | partial max [kAW][REP] | partial sum [kAW][REP] | key staging
  extern __shared__ __align__(16) float qs[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h0 = blockIdx.y * REP;
  int t = blockIdx.x, pos, seq;
  if (atoms != nullptr) {            // tokens of short atoms: kShortAtom grid slots per atom
    const int* a = atoms + 6 * (blockIdx.x / kShortAtom);
    const int i = blockIdx.x % kShortAtom;
    if (i >= a[2]) return;
    t = a[1] + i, pos = a[3] + i, seq = a[0];
  } else {
    pos = tok_pos[t], seq = tok_seq[t];
  }
  const int d8 = (d + 7) & ~7;
  float* pacc = qs + REP * d8;
  float* pm = pacc + kAW * REP * dv;
  float* pl = pm + kAW * REP;
  float* stage = pl + kAW * REP;                 // [kAW warps][32 keys][64 + pad] of T, 16-byte aligned
  for (int i = threadIdx.x; i < REP * d8; i += blockDim.x) {
    const int hh = i / d8, c = i % d8;
    qs[i] = c < d ? q[((long long)t * Hq + h0 + hh) * d + c] * scale : 0.f;
  }
  __syncthreads();
  const int g = h0 / (Hq / G);
  const int* tab = tables + (long long)seq * max_blocks;
  const int lo = first_key(pos, chunk, window);
  const bool kvec = d % 8 == 0 && kpitch % 8 == 0, vvec = dv % 4 == 0 && vpitch % 4 == 0;
  float m[REP], l[REP], acc[REP][VPL];
#pragma unroll
  for (int hh = 0; hh < REP; ++hh) {
    m[hh] = -INFINITY, l[hh] = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) acc[hh][i] = 0.f;
  }
  for (int j0 = lo + warp * 32; j0 <= pos; j0 += 32 * kAW) {
    const int j = j0 + lane;
    const int n = min(32, pos - j0 + 1);
    const long long myslot = j <= pos ? (long long)tab[j / block_size] * block_size + j % block_size : -1;
    float sc[REP];
#pragma unroll
    for (int hh = 0; hh < REP; ++hh) sc[hh] = 0.f;
    if (kvec) {
      // the tile's rows come in coalesced, 64 channels at a time, through a padded per-warp buffer; then every lane
      // reads its own row from there
      constexpr int E = 16 / (int)sizeof(T), SP = 64 + E;
      T* st = reinterpret_cast<T*>(stage) + warp * 32 * SP;
      for (int c0 = 0; c0 < d; c0 += 64) {
        const int w = min(64, d - c0), per = w / E;
        for (int i0 = 0; i0 < per; i0 += kKeyLoads) {          // kKeyLoads 16-byte loads per lane in flight
          uint4 u[kKeyLoads];
#pragma unroll
          for (int x = 0; x < kKeyLoads; ++x) {
            if (i0 + x >= per) break;
            const int i = lane + 32 * (i0 + x), r = i / per, cc = (i % per) * E;
            const long long slot = __shfl_sync(0xffffffffu, myslot, r);
            u[x] = make_uint4(0u, 0u, 0u, 0u);
            if (slot >= 0) u[x] = *reinterpret_cast<const uint4*>(kcache + slot * kpitch + g * d + c0 + cc);
          }
#pragma unroll
          for (int x = 0; x < kKeyLoads; ++x) {
            if (i0 + x >= per) break;
            const int i = lane + 32 * (i0 + x), r = i / per, cc = (i % per) * E;
            *reinterpret_cast<uint4*>(st + r * SP + cc) = u[x];
          }
        }
        __syncwarp();
        for (int cc = 0; cc < w; cc += 4) {
          const float4 x = load4_f32<T>(st + lane * SP + cc);
#pragma unroll
          for (int hh = 0; hh < REP; ++hh) {
            const float4 y = *reinterpret_cast<const float4*>(qs + hh * d8 + c0 + cc);
            sc[hh] += (y.x * x.x + y.y * x.y) + (y.z * x.z + y.w * x.w);
          }
        }
        __syncwarp();
      }
    } else if (j <= pos) {
#pragma unroll
      for (int hh = 0; hh < REP; ++hh) sc[hh] = dot_row<T>(qs + hh * d8, kcache + myslot * kpitch + g * d, d, false);
    }
    float p[REP];
#pragma unroll
    for (int hh = 0; hh < REP; ++hh) {
      float s = j <= pos ? sc[hh] : -INFINITY;
      if (dist_bias != nullptr && j <= pos)
        s += __ldg(dist_bias + (long long)(h0 + hh) * bias_len + min(pos - j, bias_len - 1));
      const float mn = fmaxf(m[hh], warp_max(s));      // finite: the tile holds at least key j0
      const float corr = expf(m[hh] - mn);             // 0 on the first tile (m = -inf)
      p[hh] = (j <= pos) ? expf(s - mn) : 0.f;
      l[hh] = l[hh] * corr + warp_sum(p[hh]);
#pragma unroll
      for (int i = 0; i < VPL; ++i) acc[hh][i] *= corr;
      m[hh] = mn;
    }
    if (vvec) {                                      // lane holds channels 128 i + 4 lane .. + 3; kValLoads keys in flight
      for (int jj = 0; jj < n; jj += kValLoads) {
        float4 v[kValLoads][VPL / 4];
#pragma unroll
        for (int u = 0; u < kValLoads; ++u) {
          const long long slot = __shfl_sync(0xffffffffu, myslot, min(jj + u, n - 1));
          const T* vr = vcache + slot * vpitch + g * dv;
#pragma unroll
          for (int i = 0; i < VPL / 4; ++i) {
            const int c = 128 * i + 4 * lane;
            v[u][i] = c < dv ? load4_f32<T>(vr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
#pragma unroll
        for (int u = 0; u < kValLoads; ++u)
#pragma unroll
          for (int hh = 0; hh < REP; ++hh) {
            const float pj = __shfl_sync(0xffffffffu, p[hh], (jj + u) & 31);      // 0 beyond the last key
#pragma unroll
            for (int i = 0; i < VPL / 4; ++i) {
              acc[hh][4 * i] += pj * v[u][i].x, acc[hh][4 * i + 1] += pj * v[u][i].y;
              acc[hh][4 * i + 2] += pj * v[u][i].z, acc[hh][4 * i + 3] += pj * v[u][i].w;
            }
          }
      }
    } else {                                         // lane holds channels lane + 32 i
      for (int jj = 0; jj < n; ++jj) {
        const long long slot = __shfl_sync(0xffffffffu, myslot, jj);
        const T* vr = vcache + slot * vpitch + g * dv;
#pragma unroll
        for (int hh = 0; hh < REP; ++hh) {
          const float pj = __shfl_sync(0xffffffffu, p[hh], jj);
#pragma unroll
          for (int i = 0; i < VPL; ++i) {
            const int c = lane + 32 * i;
            if (c < dv) acc[hh][i] += pj * to_f32<T>(vr[c]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int hh = 0; hh < REP; ++hh) {
    if (lane == 0) pm[warp * REP + hh] = m[hh], pl[warp * REP + hh] = l[hh];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c = vvec ? 128 * (i >> 2) + 4 * lane + (i & 3) : lane + 32 * i;
      if (c < dv) pacc[(warp * REP + hh) * dv + c] = acc[hh][i];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < REP * dv; idx += blockDim.x) {
    const int hh = idx / dv, c = idx % dv;
    float M = sink ? sink[h0 + hh] : -INFINITY;
#pragma unroll
    for (int w = 0; w < kAW; ++w) M = fmaxf(M, pm[w * REP + hh]);
    float L = sink ? expf(sink[h0 + hh] - M) : 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < kAW; ++w) {
      const float f = pm[w * REP + hh] == -INFINITY ? 0.f : expf(pm[w * REP + hh] - M);
      L += pl[w * REP + hh] * f;
      o += pacc[(w * REP + hh) * dv + c] * f;
    }
    float r = L > 0.f ? o / L : 0.f;
    if (gate != nullptr) r *= sigmoid_f(to_f32<T>(gate[(long long)t * gate_ld + (h0 + hh) * dv + c]));
    out[((long long)t * Hq + h0 + hh) * dv + c] = from_f32<T>(r);
  }
}

template <typename T, int REP, int VPL>
static int launch_attention_rows_v(dim3 grid, const void* q, const void* kcache, const void* vcache, const void* sink,
                                   void* out, const void* tok_seq, const void* tok_pos, const void* tables,
                                   int max_blocks, int block_size, int Hq, int G, int d, int dv, float scale,
                                   int chunk, int window, int kpitch, int vpitch, const int* atoms, const void* dist_bias,
                                   int bias_len, const void* gate, long long gate_ld, cudaStream_t s) {
  const size_t smem = (size_t)(REP * ((d + 7) & ~7) + kAW * REP * dv + 2 * kAW * REP + kAW * 32 * 68) * sizeof(float);
  cudaError_t e = cudaFuncSetAttribute(sink_attention_kernel<T, REP, VPL>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  grid.y = Hq / REP;
  sink_attention_kernel<T, REP, VPL><<<grid, 32 * kAW, smem, s>>>(
      (const float*)q, (const T*)kcache, (const T*)vcache, (const float*)sink, (T*)out, (const int*)tok_seq,
      (const int*)tok_pos, (const int*)tables, max_blocks, block_size, Hq, G, d, dv, scale, chunk, window, kpitch,
      vpitch, atoms, (const float*)dist_bias, bias_len, (const T*)gate, gate_ld);
  return SXB_OK;
}

template <typename T, int REP>
static int launch_attention_rows(dim3 grid, const void* q, const void* kcache, const void* vcache, const void* sink,
                                 void* out, const void* tok_seq, const void* tok_pos, const void* tables,
                                 int max_blocks, int block_size, int Hq, int G, int d, int dv, float scale, int chunk,
                                 int window, int kpitch, int vpitch, const int* atoms, const void* dist_bias,
                                 int bias_len, const void* gate, long long gate_ld, cudaStream_t s) {
  if (dv <= 128)
    return launch_attention_rows_v<T, REP, 4>(grid, q, kcache, vcache, sink, out, tok_seq, tok_pos, tables, max_blocks,
                                              block_size, Hq, G, d, dv, scale, chunk, window, kpitch, vpitch, atoms,
                                              dist_bias, bias_len, gate, gate_ld, s);
  return launch_attention_rows_v<T, REP, kMaxVPerLane>(grid, q, kcache, vcache, sink, out, tok_seq, tok_pos, tables,
                                                       max_blocks, block_size, Hq, G, d, dv, scale, chunk, window,
                                                       kpitch, vpitch, atoms, dist_bias, bias_len, gate, gate_ld, s);
}

// Query heads per key/value head that one CTA takes together: the largest of 8, 4, 2, 1 that divides the group.
static int attention_rows(int dtype, dim3 grid, const void* q, const void* kcache, const void* vcache,
                          const void* sink, void* out, const void* tok_seq, const void* tok_pos, const void* tables,
                          int max_blocks, int block_size, int Hq, int G, int d, int dv, float scale, int chunk,
                          int window, int kpitch, int vpitch, const int* atoms, const void* dist_bias, int bias_len,
                          const void* gate, long long gate_ld, cudaStream_t s) {
  const int group = Hq / G;
  int rc = SXB_OK;
  // (Taking fewer heads together when a decode batch leaves SMs idle was measured slower: every CTA walks all keys.)
  const int rep = group % 8 == 0 ? 8 : (group % 4 == 0 ? 4 : (group % 2 == 0 ? 2 : 1));
#define ROWS(REP)                                                                                                      \
  SEQMIX_DISPATCH(dtype, (rc = launch_attention_rows<T, REP>(grid, q, kcache, vcache, sink, out, tok_seq, tok_pos,      \
                                                              tables, max_blocks, block_size, Hq, G, d, dv, scale,      \
                                                              chunk, window, kpitch, vpitch, atoms, dist_bias,      \
                                                              bias_len, gate, gate_ld, s)))
  if (rep == 8) ROWS(8);
  else if (rep == 4) ROWS(4);
  else if (rep == 2) ROWS(2);
  else ROWS(1);
#undef ROWS
  return rc;
}

// ------------------------------------------------------------------------------------------------ short convolution
constexpr int kMaxTaps = 16;

// out[t, c] = silu(bias[c] + sum_j w[c, taps-1-j] * x[t-j, c]); x before this batch's rows comes from the slot's carried
// inputs (state [slots, taps-1, C], last row = most recent), x before the sequence's start is zero.
template <typename T>
__global__ void __launch_bounds__(256)
conv_silu_kernel(const T* __restrict__ x, long long ld, const T* __restrict__ w, const T* __restrict__ bias,
                 const T* __restrict__ state, const int* __restrict__ seq_info, const int* __restrict__ tok_seq,
                 float* __restrict__ out, int C, int taps) {
  const int t = blockIdx.x;
  const int* si = seq_info + 4 * tok_seq[t];
  const int local = t - si[0], seen = si[2];
  const T* st = state + (long long)si[3] * (taps - 1) * C;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    float a = bias ? to_f32<T>(bias[c]) : 0.f;
    for (int j = 0; j < taps; ++j) {
      const int src = local - j;
      float v = 0.f;
      if (src >= 0) v = to_f32<T>(x[(long long)(t - j) * ld + c]);
      else if (seen + src >= 0) v = to_f32<T>(st[(long long)(taps - 1 + src) * C + c]);
      a += to_f32<T>(w[(long long)c * taps + (taps - 1 - j)]) * v;
    }
    out[(long long)t * C + c] = silu_f(a);
  }
}

// The same filter for channel counts and row pitches that are multiples of 8: a thread takes 8 channels (16-byte loads
// of bf16, two of fp32) and walks kConvRows consecutive batch rows with the last TAPS-1 inputs in registers.  The window
// is loaded by the rule above at the thread's first row and at a sequence's first row in the batch, and shifted
// otherwise; the sum runs in the same order as in the scalar kernel.
constexpr int kConvRows = 8;

template <typename T>
__device__ __forceinline__ void load8_f32(const T* p, float* o);
template <>
__device__ __forceinline__ void load8_f32<float>(const float* p, float* o) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  o[0] = a.x, o[1] = a.y, o[2] = a.z, o[3] = a.w, o[4] = b.x, o[5] = b.y, o[6] = b.z, o[7] = b.w;
}
template <>
__device__ __forceinline__ void load8_f32<__nv_bfloat16>(const __nv_bfloat16* p, float* o) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) o[2 * i] = __low2float(h[i]), o[2 * i + 1] = __high2float(h[i]);
}

template <typename T, int TAPS>
__global__ void __launch_bounds__(128)
conv_silu_vec_kernel(const T* __restrict__ x, long long ld, const T* __restrict__ w, const T* __restrict__ bias,
                     const T* __restrict__ state, const int* __restrict__ seq_info, const int* __restrict__ tok_seq,
                     float* __restrict__ out, int C, int n_tokens) {
  const int c0 = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (c0 >= C) return;
  const int t0 = blockIdx.x * kConvRows, t1 = min(t0 + kConvRows, n_tokens);
  float wt[8][TAPS], b8[8], hist[TAPS][8];      // hist[j]: the input j rows back (hist[0]: the current row)
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    b8[e] = bias ? to_f32<T>(bias[c0 + e]) : 0.f;
#pragma unroll
    for (int j = 0; j < TAPS; ++j) wt[e][j] = to_f32<T>(w[(long long)(c0 + e) * TAPS + j]);
  }
  for (int t = t0; t < t1; ++t) {
    const int* si = seq_info + 4 * tok_seq[t];
    const int local = t - si[0], seen = si[2];
    if (t == t0 || local == 0) {
      const T* st = state + (long long)si[3] * (TAPS - 1) * C;
#pragma unroll
      for (int j = 1; j < TAPS; ++j) {
        const int src = local - j;
        if (src >= 0) {
          load8_f32<T>(x + (long long)(t - j) * ld + c0, hist[j]);
        } else if (seen + src >= 0) {
          load8_f32<T>(st + (long long)(TAPS - 1 + src) * C + c0, hist[j]);
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) hist[j][e] = 0.f;
        }
      }
    } else {
#pragma unroll
      for (int j = TAPS - 1; j >= 1; --j)
#pragma unroll
        for (int e = 0; e < 8; ++e) hist[j][e] = hist[j - 1][e];
    }
    load8_f32<T>(x + (long long)t * ld + c0, hist[0]);
    float o[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float a = b8[e];
#pragma unroll
      for (int j = 0; j < TAPS; ++j) a += wt[e][TAPS - 1 - j] * hist[j][e];
      o[e] = silu_f(a);
    }
    float4* op = reinterpret_cast<float4*>(out + (long long)t * C + c0);
    op[0] = make_float4(o[0], o[1], o[2], o[3]);
    op[1] = make_float4(o[4], o[5], o[6], o[7]);
  }
}

// After conv_silu of a batch: each slot keeps the last taps-1 inputs of (carried inputs ++ this batch's rows).
template <typename T>
__global__ void __launch_bounds__(256)
conv_state_update_kernel(const T* __restrict__ x, long long ld, T* __restrict__ state,
                         const int* __restrict__ seq_info, int C, int taps) {
  const int* si = seq_info + 4 * blockIdx.x;
  const int first = si[0], n = si[1], seen = si[2];
  T* st = state + (long long)si[3] * (taps - 1) * C;
  const int keep = taps - 1;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    T vals[kMaxTaps];
    for (int j = 0; j < keep; ++j) {
      const int i = n + j;           // index into carried (keep rows) ++ new (n rows)
      if (i >= keep) vals[j] = x[(long long)(first + i - keep) * ld + c];
      else vals[j] = (seen + (i - keep) >= 0) ? st[(long long)i * C + c] : from_f32<T>(0.f);
    }
    for (int j = 0; j < keep; ++j) st[(long long)j * C + c] = vals[j];
  }
}

// x[t, col0 + h*dim .. +dim] <- x * mult / sqrt(sum(x^2) + eps); one warp per (token, head).
__global__ void __launch_bounds__(128)
unit_norm_heads_kernel(float* __restrict__ x, long long ld, int col0, int n_heads, int dim, float mult, float eps,
                       int n_tokens) {
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (idx >= n_tokens * n_heads) return;
  float* p = x + (long long)(idx / n_heads) * ld + col0 + (idx % n_heads) * dim;
  float ss = 0.f;
  for (int c = lane; c < dim; c += 32) ss += p[c] * p[c];
  ss = warp_sum(ss);
  const float inv = mult / sqrtf(ss + eps);
  for (int c = lane; c < dim; c += 32) p[c] *= inv;
}

// mode 0 (delta rule):  beta = sigmoid(b_raw), decay = exp(-exp(A_log) * softplus(a_raw + dt_bias))
// mode 1 (state space): dt = softplus(a_raw + dt_bias), beta = dt, decay = exp(-exp(A_log) * dt)
template <typename T>
__global__ void __launch_bounds__(256)
recurrence_gates_kernel(const T* __restrict__ a_raw, const T* __restrict__ b_raw, long long ld,
                        const float* __restrict__ A_log, const float* __restrict__ dt_bias, float* __restrict__ decay,
                        float* __restrict__ beta, int H, int n_tokens, int mode) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_tokens * H) return;
  const int t = i / H, h = i % H;
  const float dt = softplus_f(to_f32<T>(a_raw[(long long)t * ld + h]) + dt_bias[h]);
  decay[i] = expf(-expf(A_log[h]) * dt);
  beta[i] = mode == 0 ? sigmoid_f(to_f32<T>(b_raw[(long long)t * ld + h])) : dt;
}

// Decay per (head, key channel) pair:  decay[t, h, c] = exp(-exp(A_log[h]) * softplus(a_raw[t, h n + c] + dt_bias[h n + c])),
// beta[t, h] = sigmoid(b_raw[t, h]).  a_raw rows of pitch lda hold H n channels, b_raw rows of pitch ldb hold H.
template <typename T>
__global__ void __launch_bounds__(256)
channel_decay_gates_kernel(const T* __restrict__ a_raw, long long lda, const T* __restrict__ b_raw, long long ldb,
                           const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                           float* __restrict__ decay, float* __restrict__ beta, int H, int n, long long total) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int Hn = H * n;
  const long long t = i / Hn;
  const int c = (int)(i % Hn), h = c / n;
  const float dt = softplus_f(to_f32<T>(a_raw[t * lda + c]) + dt_bias[c]);
  decay[i] = expf(-expf(A_log[h]) * dt);
  if (c < H) beta[t * H + c] = sigmoid_f(to_f32<T>(b_raw[t * ldb + c]));
}

// ------------------------------------------------------------------------------------------------ recurrence
// State per (slot, head): dv columns of n floats, stored [dv][n].  Each output column evolves on its own:
//   s <- a s;  u = b (v_c - [delta] s.k);  s <- s + k u;  o_c = s.q (+ D v_c)
// A column is held by LPC = 8 lanes (the n-vector as 16-byte chunks, chunk i on lane i mod LPC), 128 / LPC columns per
// CTA; the CTA walks its sequence's rows in order, staging k and q of TB tokens at a time in shared memory.  (Spreading
// a column over a whole warp gives a long sequence four times as many warps, but was measured slower: the work per SM
// is the same and the longer shuffle trees add instructions.)  The products run as packed pairs (fma.f32x2).
constexpr int kRecThreads = 128, kTB = 8;

template <int R, bool DELTA, int LPC, bool CHAN>
__global__ void __launch_bounds__(kRecThreads)
linear_recurrence_kernel(const float* __restrict__ kvec, const float* __restrict__ qvec, long long ldkq,
                         const float* __restrict__ val, long long ldv, const float* __restrict__ decay,
                         const float* __restrict__ beta, const float* __restrict__ skip, float* __restrict__ state,
                         float* __restrict__ out, const int* __restrict__ seq_info, int H, int G, int n, int dv) {
  // Lane l of a column holds the float4 chunks l, l + LPC, l + 2 LPC, ... of the column's n-vector (padded with zeros
  // to NP = LPC R), so k, q and the state move as 16-byte words without bank conflicts.  Two staging buffers, each
  // k [TB][NP] | q [TB][NP] | v [TB][COLS] | decay [TB] | beta [TB]: the next TB tokens are copied in (cp.async) while
  // the current ones are walked.  CHAN: the decay is a vector over the key channels (decay [rows, H n]) and follows the
  // scalars as one more [TB][NP] block; the state is multiplied by it chunk by chunk before the delta rule's product.
  constexpr int NP = R * LPC, R4 = R / 4, COLS = kRecThreads / LPC;
  extern __shared__ __align__(16) float sm[];
  constexpr int stage = (CHAN ? 3 : 2) * kTB * NP + kTB * COLS + 2 * kTB;
  const int* si = seq_info + 4 * blockIdx.z;
  const int first = si[0], rows = si[1], seen = si[2], slot = si[3];
  const int h = blockIdx.y, g = h / (H / G);
  const int lc = threadIdx.x / LPC, l = threadIdx.x % LPC;
  const int col = blockIdx.x * COLS + lc;
  const bool live = col < dv;
  for (int i = threadIdx.x; i < 2 * stage; i += blockDim.x) sm[i] = 0.f;      // the padding stays zero
  float* sp = state + (((long long)slot * H + h) * dv + (live ? col : 0)) * n;
  const bool n4 = (n & 3) == 0;
  const bool wide_copy = n4 && (ldkq & 3) == 0 && ((reinterpret_cast<uintptr_t>(kvec) & 15) == 0) &&
                         ((reinterpret_cast<uintptr_t>(qvec) & 15) == 0);
  float2 S[R / 2];
#pragma unroll
  for (int r4 = 0; r4 < R4; ++r4) {
    const int i = (r4 * LPC + l) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live && seen > 0) {
      if (n4 && i < n) {
        v = *reinterpret_cast<const float4*>(sp + i);
      } else {
        if (i < n) v.x = sp[i];
        if (i + 1 < n) v.y = sp[i + 1];
        if (i + 2 < n) v.z = sp[i + 2];
        if (i + 3 < n) v.w = sp[i + 3];
      }
    }
    S[2 * r4] = make_float2(v.x, v.y), S[2 * r4 + 1] = make_float2(v.z, v.w);
  }
  const float D = skip ? skip[h] : 0.f;
  __syncthreads();

  auto stage_in = [&](int buf, int t0) {
    float* sk = sm + buf * stage;
    float* sq = sk + kTB * NP;
    float* sv = sq + kTB * NP;
    float* sa = sv + kTB * COLS;
    float* sb = sa + kTB;
    float* sg = sb + kTB;
    const int nt = min(kTB, rows - t0);
    if (CHAN) {
      const long long Hn = (long long)H * n;
      if (n4) {
        const int nq4 = n >> 2;
        for (int i = threadIdx.x; i < nt * nq4; i += blockDim.x) {
          const int tt = i / nq4, c = (i % nq4) * 4;
          __pipeline_memcpy_async(sg + tt * NP + c, decay + (long long)(first + t0 + tt) * Hn + (long long)h * n + c, 16);
        }
      } else {
        for (int i = threadIdx.x; i < nt * n; i += blockDim.x) {
          const int tt = i / n, c = i % n;
          __pipeline_memcpy_async(sg + tt * NP + c, decay + (long long)(first + t0 + tt) * Hn + (long long)h * n + c, 4);
        }
      }
    }
    if (wide_copy) {
      const int nq4 = n >> 2;
      for (int i = threadIdx.x; i < nt * nq4; i += blockDim.x) {
        const int tt = i / nq4, c = (i % nq4) * 4;
        const long long row = first + t0 + tt;
        __pipeline_memcpy_async(sk + tt * NP + c, kvec + row * ldkq + g * n + c, 16);
        __pipeline_memcpy_async(sq + tt * NP + c, qvec + row * ldkq + g * n + c, 16);
      }
    } else {
      for (int i = threadIdx.x; i < nt * n; i += blockDim.x) {
        const int tt = i / n, c = i % n;
        const long long row = first + t0 + tt;
        __pipeline_memcpy_async(sk + tt * NP + c, kvec + row * ldkq + g * n + c, 4);
        __pipeline_memcpy_async(sq + tt * NP + c, qvec + row * ldkq + g * n + c, 4);
      }
    }
    for (int i = threadIdx.x; i < nt * COLS; i += blockDim.x) {
      const int c = min((int)blockIdx.x * COLS + i % COLS, dv - 1);
      __pipeline_memcpy_async(sv + i, val + (long long)(first + t0 + i / COLS) * ldv + h * dv + c, 4);
    }
    for (int i = threadIdx.x; i < nt; i += blockDim.x) {
      if (!CHAN) __pipeline_memcpy_async(sa + i, decay + (long long)(first + t0 + i) * H + h, 4);
      __pipeline_memcpy_async(sb + i, beta + (long long)(first + t0 + i) * H + h, 4);
    }
    __pipeline_commit();
  };

  stage_in(0, 0);
  int buf = 0;
  for (int t0 = 0; t0 < rows; t0 += kTB, buf ^= 1) {
    const int nt = min(kTB, rows - t0);
    const bool more = t0 + kTB < rows;
    if (more) stage_in(buf ^ 1, t0 + kTB);
    if (more) __pipeline_wait_prior(1);
    else __pipeline_wait_prior(0);
    __syncthreads();
    const float* sk = sm + buf * stage;
    const float* sq = sk + kTB * NP;
    const float* sv = sq + kTB * NP;
    const float* sa = sv + kTB * COLS;
    const float* sb = sa + kTB;
    const float* sg = sb + kTB;
    // One token.  A full group of TB tokens is walked by straight-line code, so the loads of k and q and the read-out
    // reductions of neighbouring tokens overlap the serial part (the state update, and the dot product before it for
    // the delta rule).
    struct Tok {                      // one token's operands, loaded one token ahead of their use
      float a, b, v;
      float4 k[R4], q[R4], g[CHAN ? R4 : 1];
    };
    auto fetch = [&](int tt) {
      Tok t;
      t.a = CHAN ? 1.f : sa[tt], t.b = sb[tt], t.v = sv[tt * COLS + lc];
      const float4* kk = reinterpret_cast<const float4*>(sk + tt * NP) + l;
      const float4* qq = reinterpret_cast<const float4*>(sq + tt * NP) + l;
#pragma unroll
      for (int r4 = 0; r4 < R4; ++r4) t.k[r4] = kk[r4 * LPC], t.q[r4] = qq[r4 * LPC];
      if (CHAN) {
        const float4* gg = reinterpret_cast<const float4*>(sg + tt * NP) + l;
#pragma unroll
        for (int r4 = 0; r4 < R4; ++r4) t.g[r4] = gg[r4 * LPC];
      }
      return t;
    };
    auto step = [&](const Tok& t, float& o_lane) {
      const float a = t.a, b = t.b, v = t.v;
      const float4* k4 = t.k;
      float u = b * v;
      if (CHAN) {                      // the decayed state enters the product below: decay first, a stays 1
#pragma unroll
        for (int r4 = 0; r4 < R4; ++r4) {
          S[2 * r4] = __fmul2_rn(S[2 * r4], make_float2(t.g[r4].x, t.g[r4].y));
          S[2 * r4 + 1] = __fmul2_rn(S[2 * r4 + 1], make_float2(t.g[r4].z, t.g[r4].w));
        }
      }
      if (DELTA) {                     // (a S)^T k = a (S^T k): the decay is folded into the update below
        float2 d01 = make_float2(0.f, 0.f), d23 = make_float2(0.f, 0.f);
#pragma unroll
        for (int r4 = 0; r4 < R4; ++r4) {
          d01 = __ffma2_rn(S[2 * r4], make_float2(k4[r4].x, k4[r4].y), d01);
          d23 = __ffma2_rn(S[2 * r4 + 1], make_float2(k4[r4].z, k4[r4].w), d23);
        }
        float dot = (d01.x + d01.y) + (d23.x + d23.y);
#pragma unroll
        for (int o = 1; o < LPC; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        u = b * (v - a * dot);
      }
      const float2 a2 = make_float2(a, a), u2 = make_float2(u, u);
      float2 o01 = make_float2(0.f, 0.f), o23 = make_float2(0.f, 0.f);
#pragma unroll
      for (int r4 = 0; r4 < R4; ++r4) {
        const float4 q4 = t.q[r4];
        S[2 * r4] = __ffma2_rn(make_float2(k4[r4].x, k4[r4].y), u2, CHAN ? S[2 * r4] : __fmul2_rn(S[2 * r4], a2));
        S[2 * r4 + 1] = __ffma2_rn(make_float2(k4[r4].z, k4[r4].w), u2,
                                   CHAN ? S[2 * r4 + 1] : __fmul2_rn(S[2 * r4 + 1], a2));
        o01 = __ffma2_rn(S[2 * r4], make_float2(q4.x, q4.y), o01);
        o23 = __ffma2_rn(S[2 * r4 + 1], make_float2(q4.z, q4.w), o23);
      }
      o_lane = (o01.x + o01.y) + (o23.x + o23.y);       // this lane's part of the read-out
    };
    if (nt == kTB) {
      // the read-outs of the group are summed over the column's lanes together, off the serial path: TB independent
      // shuffle trees, then lane t of the column writes token t
      static_assert(LPC == kTB, "lane t of a column writes token t of the group");
      float op[kTB];
      Tok cur = fetch(0);
#pragma unroll
      for (int tt = 0; tt < kTB; ++tt) {
        const Tok nxt = fetch(tt + 1 < kTB ? tt + 1 : tt);
        step(cur, op[tt]);
        cur = nxt;
      }
#pragma unroll
      for (int x = 1; x < LPC; x <<= 1)
#pragma unroll
        for (int tt = 0; tt < kTB; ++tt) op[tt] += __shfl_xor_sync(0xffffffffu, op[tt], x);
      float mine = op[0];
#pragma unroll
      for (int tt = 1; tt < kTB; ++tt) mine = (l == tt) ? op[tt] : mine;
      if (live) out[(long long)(first + t0 + l) * H * dv + h * dv + col] = mine + D * sv[l * COLS + lc];
    } else {
      for (int tt = 0; tt < nt; ++tt) {
        float o;
        step(fetch(tt), o);
#pragma unroll
        for (int x = 1; x < LPC; x <<= 1) o += __shfl_xor_sync(0xffffffffu, o, x);
        if (live && l == 0) out[(long long)(first + t0 + tt) * H * dv + h * dv + col] = o + D * sv[tt * COLS + lc];
      }
    }
    __syncthreads();          // the buffer just walked is the target of the next iteration's copies
  }
  if (live) {
#pragma unroll
    for (int r4 = 0; r4 < R4; ++r4) {
      const int i = (r4 * LPC + l) * 4;
      if (n4 && i < n) {
        *reinterpret_cast<float4*>(sp + i) = make_float4(S[2 * r4].x, S[2 * r4].y, S[2 * r4 + 1].x, S[2 * r4 + 1].y);
      } else {
        if (i < n) sp[i] = S[2 * r4].x;
        if (i + 1 < n) sp[i + 1] = S[2 * r4].y;
        if (i + 2 < n) sp[i + 2] = S[2 * r4 + 1].x;
        if (i + 3 < n) sp[i + 3] = S[2 * r4 + 1].y;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------ gated group norm
// One CTA per (token, group of `gs` channels).  gate_first: z = y * silu(gate); out = z / rms(z) * w.
// else: out = y / rms(y) * w * silu(gate).  w has `wlen` entries and repeats along the row.
template <typename T>
__global__ void __launch_bounds__(128)
group_norm_gate_kernel(const float* __restrict__ y, const T* __restrict__ gate, long long ldg,
                       const T* __restrict__ w, int wlen, T* __restrict__ out, int C, int gs, float eps,
                       int gate_first) {
  __shared__ float red[32];
  const int t = blockIdx.x, c0 = blockIdx.y * gs;
  const float* yr = y + (long long)t * C + c0;
  const T* gr = gate + (long long)t * ldg + c0;
  const bool sigm = (gate_first & 2) != 0;      // bit 1: the gate is sigmoid(gate) instead of silu(gate)
  gate_first &= 1;
  float ss = 0.f;
  for (int c = threadIdx.x; c < gs; c += blockDim.x) {
    float v = yr[c];
    if (gate_first) v *= sigm ? sigmoid_f(to_f32<T>(gr[c])) : silu_f(to_f32<T>(gr[c]));
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)gs + eps);
  for (int c = threadIdx.x; c < gs; c += blockDim.x) {
    const float sg = sigm ? sigmoid_f(to_f32<T>(gr[c])) : silu_f(to_f32<T>(gr[c]));
    const float wv = to_f32<T>(w[(c0 + c) % wlen]);
    const float v = gate_first ? yr[c] * sg * inv * wv : yr[c] * inv * wv * sg;
    out[(long long)t * C + c0 + c] = from_f32<T>(v);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
gated_act_rows_kernel(const T* __restrict__ in, T* __restrict__ out, long long total, int F, int act, float limit) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long r = i / F;
  const int c = (int)(i % F);
  float gte = to_f32<T>(in[r * 2 * F + c]), up = to_f32<T>(in[r * 2 * F + F + c]);
  float a;
  if (act == 5) {          // clamped: a = min(gate, L), b = max(-L, min(up, L)); a sigmoid(1.702 a) (1 + b)
    gte = fminf(gte, limit);
    up = fminf(fmaxf(up, -limit), limit) + 1.f;
    a = gte * sigmoid_f(1.702f * gte);
  } else if (act == 2) {
    a = 0.5f * gte * (1.f + tanhf(0.7978845608028654f * (gte + 0.044715f * gte * gte * gte)));
  } else if (act == 3) {
    a = silu_f(gte);
  } else if (act == 1) {
    a = fmaxf(gte, 0.f);
  } else {
    a = gte;
  }
  out[i] = from_f32<T>(a * up);
}


__device__ __forceinline__ float gated_act_value(float gte, float up, int act, float limit) {
  if (act == 5) {
    gte = fminf(gte, limit);
    return gte * sigmoid_f(1.702f * gte) * (fminf(fmaxf(up, -limit), limit) + 1.f);
  }
  float a = gte;
  if (act == 2) a = 0.5f * gte * (1.f + tanhf(0.7978845608028654f * (gte + 0.044715f * gte * gte * gte)));
  else if (act == 3) a = silu_f(gte);
  else if (act == 1) a = fmaxf(gte, 0.f);
  return a * up;
}

// The same with VEC consecutive channels per thread (16-byte accesses): F a multiple of VEC, rows 16-byte aligned.
template <typename T, int VEC>
__global__ void __launch_bounds__(256)
gated_act_rows_vec_kernel(const T* __restrict__ in, T* __restrict__ out, long long nvec, int fvec, int act, float limit) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nvec) return;
  const long long r = i / fvec;
  const int c = (int)(i % fvec) * VEC;
  const int F = fvec * VEC;
  struct alignas(16) Pack { T v[VEC]; };
  const Pack g = *reinterpret_cast<const Pack*>(in + r * 2 * F + c);
  const Pack u = *reinterpret_cast<const Pack*>(in + r * 2 * F + F + c);
  Pack o;
#pragma unroll
  for (int j = 0; j < VEC; ++j) o.v[j] = from_f32<T>(gated_act_value(to_f32<T>(g.v[j]), to_f32<T>(u.v[j]), act, limit));
  *reinterpret_cast<Pack*>(out + r * F + c) = o;
}

// ------------------------------------------------------------------------------------------------ post-norm layers
// Layers of the form  x <- x + scale (.) (sublayer(x + conv(x)) / rms * gain):  the sublayer reads the fp32 stream
// through a short causal filter with a skip path, its output is normalised with ONE gain for all channels and scaled
// per channel before it joins the stream; the stream a layer hands on may be a learned mixture of the embedding and
// all layers' results so far.

// out[t, c] = x[t, c] + sum_j w[c, taps-1-j] x[t-j, c]; x fp32, rows before this batch from the slot's carried inputs
// (state fp32 [slots, taps-1, C], last row = most recent), rows before the sequence's start are zero.
template <typename T>
__global__ void __launch_bounds__(256)
conv_residual_kernel(const float* __restrict__ x, const T* __restrict__ w, const float* __restrict__ state,
                     const int* __restrict__ seq_info, const int* __restrict__ tok_seq, T* __restrict__ out, int C,
                     int taps) {
  const int t = blockIdx.x;
  const int* si = seq_info + 4 * tok_seq[t];
  const int local = t - si[0], seen = si[2];
  const float* st = state + (long long)si[3] * (taps - 1) * C;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    const T* wc = w + (long long)c * taps;
    const float cur = x[(long long)t * C + c];
    float acc = 0.f;
    for (int j = taps - 1; j >= 1; --j) {            // oldest input first
      const int src = local - j;
      float v = 0.f;
      if (src >= 0) v = x[(long long)(t - j) * C + c];
      else if (seen + src >= 0) v = st[(long long)(taps - 1 + src) * C + c];
      acc += to_f32<T>(wc[taps - 1 - j]) * v;
    }
    acc += to_f32<T>(wc[taps - 1]) * cur;
    out[(long long)t * C + c] = from_f32<T>(cur + acc);
  }
}

// One CTA per row: v = x_in + ls (.) (y / rms(y) * gain) -> x_out (may be x_in); with mix_out:
// mix_out = sum_{j < n_prev} mixw[j] stack[j] + mixw[n_prev] v  (stack[j] = fp32 rows at stack + j * stack_stride).
template <typename T>
__global__ void __launch_bounds__(256)
post_norm_mix_kernel(const float* __restrict__ x_in, const T* __restrict__ y, const float* __restrict__ gain,
                     const float* __restrict__ ls, float* __restrict__ x_out, const float* __restrict__ stack,
                     long long stack_stride, int n_prev, const float* __restrict__ mixw, float* __restrict__ mix_out,
                     int width, float eps) {
  __shared__ float red[32];
  const long long base = (long long)blockIdx.x * width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = to_f32<T>(y[base + c]);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)width + eps);
  const float g = gain[0];
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = x_in[base + c] + to_f32<T>(y[base + c]) * inv * g * ls[c];
    x_out[base + c] = v;
    if (mix_out != nullptr) {
      float m = 0.f;
      for (int j = 0; j < n_prev; ++j) m += mixw[j] * stack[j * stack_stride + base + c];
      mix_out[base + c] = m + mixw[n_prev] * v;
    }
  }
}

// out[i] = x[rows[i]] / rms * gain (one gain for all channels); rows null: every row in order.
template <typename T>
__global__ void __launch_bounds__(256)
rms_scale_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ gain,
                      T* __restrict__ out, int width, float eps) {
  __shared__ float red[32];
  const float* r = x + (long long)(rows ? rows[blockIdx.x] : blockIdx.x) * width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) ss += r[c] * r[c];
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)width + eps);
  const float g = gain[0];
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    out[(long long)blockIdx.x * width + c] = from_f32<T>(r[c] * inv * g);
}

// out [rows, n] = x[:, :n] / rms * w for rows of pitch ld.
template <typename T>
__global__ void __launch_bounds__(128)
rms_norm_slice_kernel(const T* __restrict__ x, long long ld, const T* __restrict__ w, T* __restrict__ out, int n,
                      float eps) {
  __shared__ float red[32];
  const T* r = x + (long long)blockIdx.x * ld;
  float ss = 0.f;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    const float v = to_f32<T>(r[c]);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)n + eps);
  for (int c = threadIdx.x; c < n; c += blockDim.x)
    out[(long long)blockIdx.x * n + c] = from_f32<T>(to_f32<T>(r[c]) * inv * to_f32<T>(w[c]));
}

// out = act(in + bias) for rows of any width; act as in gated_act_rows plus 4 = relu(z)^2.
__device__ __forceinline__ float act_f(float z, int act) {
  if (act == 4) {
    const float r = fmaxf(z, 0.f);
    return r * r;
  }
  if (act == 2) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  if (act == 3) return silu_f(z);
  if (act == 1) return fmaxf(z, 0.f);
  return z;
}

template <typename T>
__global__ void __launch_bounds__(256)
bias_act_rows_kernel(const T* __restrict__ in, const T* __restrict__ bias, T* __restrict__ out, long long total, int F,
                     int act) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  out[i] = from_f32<T>(act_f(to_f32<T>(in[i]) + (bias ? to_f32<T>(bias[i % F]) : 0.f), act));
}

// 16 bytes per thread and access: widths that are multiples of 16 / sizeof(T), 16-byte aligned pointers.
template <typename T>
__global__ void __launch_bounds__(256)
bias_act_rows_vec_kernel(const T* __restrict__ in, const T* __restrict__ bias, T* __restrict__ out, long long total_vec,
                         int F, int act) {
  constexpr int E = 16 / (int)sizeof(T);
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total_vec) return;
  uint4 u = reinterpret_cast<const uint4*>(in)[i];
  T* v = reinterpret_cast<T*>(&u);
  uint4 ub = make_uint4(0u, 0u, 0u, 0u);
  if (bias) ub = *reinterpret_cast<const uint4*>(bias + (i * E) % F);
  const T* b = reinterpret_cast<const T*>(&ub);
#pragma unroll
  for (int e = 0; e < E; ++e) v[e] = from_f32<T>(act_f(to_f32<T>(v[e]) + (bias ? to_f32<T>(b[e]) : 0.f), act));
  reinterpret_cast<uint4*>(out)[i] = u;
}

// ------------------------------------------------------------------------------------------------ latent attention
// Keys and values are up-projections of one latent vector per token, so the cache holds the normalised latent (r
// channels) followed by one rotated key part (rot channels) that all heads share; a query head meets them as
// [q_abs | q_rot], q_abs its unrotated part carried through the key up-projection.  One CTA per token:
//   cache[slot] = [ latent / rms * w_norm | rope(k_rot) ],  q_out[t, h] = [ q_abs[t, h] | rope(q[t, h, dim:]) ]  (fp32)
// rope turns the pairs (2i, 2i+1), i < rot_dims / 2, by pos * inv_freq[i] and multiplies them by amp (cos and sin both
// carry the factor); channels from rot_dims on pass unchanged.
template <typename T>
__device__ __forceinline__ void rope_pairs(const T* __restrict__ src, int rot, int rot_dims, float pos,
                                           const float* __restrict__ inv_freq, int lane, int stride, float* dst32,
                                           T* dstT, float amp) {
  for (int i = lane; i < rot; i += stride) {
    float v = to_f32<T>(src[i]);
    if (i < rot_dims) {
      float sn, cs;
      sincosf(pos * inv_freq[i >> 1], &sn, &cs);
      sn *= amp, cs *= amp;
      const float other = to_f32<T>(src[i ^ 1]);
      v = (i & 1) ? v * cs + other * sn : v * cs - other * sn;
    }
    if (dst32) dst32[i] = v;
    else dstT[i] = from_f32<T>(v);
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
latent_qk_prepare_kernel(const T* __restrict__ qfull, long long ldq, const T* __restrict__ qabs, long long qa_tok,
                         long long qa_head, const T* __restrict__ kv, long long ldkv, const T* __restrict__ w_norm,
                         const float* __restrict__ inv_freq, float* __restrict__ q_out, T* __restrict__ cache,
                         const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                         const int* __restrict__ tables, int max_blocks, int block_size, int H, int dim, int rot, int r,
                         int rot_dims, float eps, float amp) {
  __shared__ float red[32];
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int p = tok_pos[t];
  const float pos = (float)p;
  const long long page = tables[(long long)tok_seq[t] * max_blocks + p / block_size];
  T* crow = cache + (page * block_size + p % block_size) * (long long)(r + rot);
  const T* kr = kv + (long long)t * ldkv;
  float ss = 0.f;
  for (int c = threadIdx.x; c < r; c += blockDim.x) {
    const float v = to_f32<T>(kr[c]);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)r + eps);
  for (int c = threadIdx.x; c < r; c += blockDim.x)
    crow[c] = from_f32<T>(to_f32<T>(kr[c]) * inv * to_f32<T>(w_norm[c]));
  rope_pairs<T>(kr + r, rot, rot_dims, pos, inv_freq, threadIdx.x, blockDim.x, nullptr, crow + r, amp);
  const int d = r + rot;
  for (int h = warp; h < H; h += nw) {
    float* qo = q_out + ((long long)t * H + h) * d;
    const T* qa = qabs + (long long)t * qa_tok + (long long)h * qa_head;
    for (int c = lane; c < r; c += 32) qo[c] = to_f32<T>(qa[c]);
    rope_pairs<T>(qfull + (long long)t * ldq + (long long)h * (dim + rot) + dim, rot, rot_dims, pos, inv_freq, lane, 32,
                  qo + r, nullptr, amp);
  }
}

// ------------------------------------------------------------------------------------------------ matrix-memory LSTM
// Per head, with log gates i, f and a running maximum m (0 for a new sequence):
//   m_t = max(f_t + m_(t-1), i_t);  S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T;  n_t likewise with k_t;
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
// The normaliser n rides along as one more value channel that is always 1, so the recurrence itself is
// linear_recurrence with decay = exp(f + m_prev - m), write strength = exp(i - m) and dv + 1 channels.

// buf fp32 [rows, 2 H n + H (dv + 1)] = [ q * qscale | k | per head (v, 1) ] from projection rows [q | k | v | ...].
template <typename T>
__global__ void __launch_bounds__(256)
mlstm_prepare_kernel(const T* __restrict__ proj, long long ld, float* __restrict__ buf, int H, int n, int dv,
                     float qscale) {
  const int t = blockIdx.x;
  const T* row = proj + (long long)t * ld;
  const int nq = H * n, wide = 2 * nq + H * (dv + 1);
  float* o = buf + (long long)t * wide;
  for (int c = threadIdx.x; c < wide; c += blockDim.x) {
    float v;
    if (c < nq) v = to_f32<T>(row[c]) * qscale;
    else if (c < 2 * nq) v = to_f32<T>(row[c]);
    else {
      const int h = (c - 2 * nq) / (dv + 1), e = (c - 2 * nq) % (dv + 1);
      v = e == dv ? 1.f : to_f32<T>(row[2 * nq + h * dv + e]);
    }
    o[c] = v;
  }
}

// One CTA per (sequence, head): gates of blockDim.x tokens at a time, the running maximum through a scan of the maps
// m -> max(m + f, i) (within the warps by shuffles, across them through shared memory).
// i = cap tanh((raw_i + b_i) / cap), f = logsigmoid(cap tanh((raw_f + b_f) / cap)).
constexpr int kScanThreads = 512;

template <typename T>
__global__ void __launch_bounds__(kScanThreads)
mlstm_gate_scan_kernel(const T* __restrict__ raw_i, const T* __restrict__ raw_f, long long ld,
                       const float* __restrict__ bias_i, const float* __restrict__ bias_f, float cap,
                       float* __restrict__ mstate, float* __restrict__ decay, float* __restrict__ beta,
                       float* __restrict__ mt, const int* __restrict__ seq_info, int H) {
  __shared__ float wa[kScanThreads / 32], wb[kScanThreads / 32], carry;
  const int* si = seq_info + 4 * blockIdx.x;
  const int first = si[0], rows = si[1], seen = si[2], slot = si[3];
  const int h = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  float m = seen > 0 ? mstate[(long long)slot * H + h] : 0.f;
  const float bi = bias_i[h], bf = bias_f[h];
  for (int t0 = 0; t0 < rows; t0 += blockDim.x) {
    const int t = t0 + threadIdx.x;
    const bool valid = t < rows;
    float ig = -INFINITY, fg = 0.f;                 // rows past the end hold the identity map
    if (valid) {
      const long long o = (long long)(first + t) * ld + h;
      ig = cap * tanhf((to_f32<T>(raw_i[o]) + bi) / cap);
      const float fr = cap * tanhf((to_f32<T>(raw_f[o]) + bf) / cap);
      fg = fminf(fr, 0.f) - log1pf(expf(-fabsf(fr)));
    }
    float a = fg, b = ig;                           // the map m -> max(m + a, b) of this warp's tokens up to t
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const float ap = __shfl_up_sync(0xffffffffu, a, off), bp = __shfl_up_sync(0xffffffffu, b, off);
      if (lane >= off) {
        b = fmaxf(bp + a, b);
        a = ap + a;
      }
    }
    if (lane == 31) wa[warp] = a, wb[warp] = b;
    __syncthreads();
    float pa = 0.f, pb = -INFINITY;                 // the map of the warps before this one
    for (int w = 0; w < warp; ++w) {
      pb = fmaxf(pb + wa[w], wb[w]);
      pa += wa[w];
    }
    const float mstart = fmaxf(m + pa, pb);         // the maximum after the last token of the warps before
    const float mcur = fmaxf(mstart + a, b);
    float mprev = __shfl_up_sync(0xffffffffu, mcur, 1);
    if (lane == 0) mprev = mstart;
    if (valid) {
      const long long o = (long long)(first + t) * H + h;
      decay[o] = expf(fg + mprev - mcur);
      beta[o] = expf(ig - mcur);
      mt[o] = mcur;
    }
    if (threadIdx.x == blockDim.x - 1) carry = mcur;
    __syncthreads();
    m = carry;
  }
  (void)nw;
  if (threadIdx.x == 0) mstate[(long long)slot * H + h] = m;
}

// One warp per (token, head): o fp32 [rows, H (dv + 1)] -> out = unit_rms(o[:dv] / (max(|o[dv]|, exp(-m)) + 1e-6)) * w *
// sigmoid(gate).
template <typename T>
__global__ void __launch_bounds__(128)
mlstm_output_kernel(const float* __restrict__ o, const float* __restrict__ mt, const T* __restrict__ gate,
                    long long ldg, const T* __restrict__ w, T* __restrict__ out, int n_tokens, int H, int dv,
                    float eps) {
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (idx >= n_tokens * H) return;
  const int t = idx / H, h = idx % H;
  const float* r = o + ((long long)t * H + h) * (dv + 1);
  const float den = fmaxf(fabsf(r[dv]), expf(-mt[idx])) + 1e-6f;
  float ss = 0.f;
  for (int c = lane; c < dv; c += 32) {
    const float v = r[c] / den;
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)dv + eps);
  for (int c = lane; c < dv; c += 32) {
    const float g = sigmoid_f(to_f32<T>(gate[(long long)t * ldg + h * dv + c]));
    out[(long long)t * H * dv + h * dv + c] = from_f32<T>(r[c] / den * inv * to_f32<T>(w[h * dv + c]) * g);
  }
}

}  // namespace seqmix
}  // namespace sxb

using namespace sxb;
using namespace sxb::seqmix;

/* out fp32 [n_tokens, width] = table[ids[t]] * scale + p, p[2i] = sin(pos * base^(-2i/width)), p[2i+1] = cos(same);
 * base <= 0: p = 0.  table: `dtype` [vocab, width]. */
SXB_API int sxb_embed_sinusoid(const void* ids, const void* pos, const void* table, void* out, int n_tokens, int width,
                               float scale, float base, int dtype, void* stream) {
  if (n_tokens <= 0) return SXB_OK;
  SEQMIX_DISPATCH(dtype, (embed_sinusoid_kernel<T><<<n_tokens, 256, 0, (cudaStream_t)stream>>>(
                             (const int*)ids, (const int*)pos, (const T*)table, (float*)out, width, scale, base)));
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}

/* Per row of the fp32 residual [rows, width]: if y: residual += mult * y / rms(y) * w_post (without w_post: += mult * y),
 * the addend times y_scale per channel if given; if extra (fp32): residual += extra; if w_pre: out = residual /
 * rms(residual) * (w_add + w_pre) (out without w_pre: the residual in `dtype`).  y, w_post, w_pre, y_scale, out are
 * `dtype`; any of the parts may be absent (null). */
SXB_API int sxb_resid_norm_step(void* resid, const void* y, const void* w_post, const void* extra, const void* w_pre,
                                void* out, long long rows, int width, float eps, float mult, int dtype,
                                const void* y_scale, float w_add, void* stream) {
  if (rows <= 0) return SXB_OK;
  if ((y == nullptr && w_post != nullptr) || (w_pre != nullptr && out == nullptr)) return SXB_ERR_BAD_ARG;
  SEQMIX_DISPATCH(dtype, (resid_norm_step_kernel<T><<<(unsigned)rows, 256, 0, (cudaStream_t)stream>>>(
                             (float*)resid, (const T*)y, (const T*)w_post, (const float*)extra, (const T*)w_pre,
                             (T*)out, width, eps, mult, (const T*)y_scale, w_add)));
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}

/* Fused projection rows qkv [n_tokens, ld] = [Hq*d | G*d | G*dv] (+ bias): q and k heads divided by their root mean
 * square (normalize != 0), q -> q_out fp32 [n_tokens, Hq, d], k -> kcache [pages, block_size, G, d], v -> vcache
 * [pages, block_size, G, dv] at each token's (page, offset). */
SXB_API int sxb_qk_norm_append(const void* qkv, long long ld, const void* bias, void* q_out, void* kcache, void* vcache,
                               const void* tok_seq, const void* tok_pos, const void* tables, int n_tokens,
                               int max_blocks, int block_size, int Hq, int G, int d, int dv, float eps, int normalize,
                               int dtype, void* stream) {
  if (n_tokens <= 0) return SXB_OK;
  SEQMIX_DISPATCH(dtype, (qk_norm_append_kernel<T><<<n_tokens, 128, 0, (cudaStream_t)stream>>>(
                             (const T*)qkv, ld, (const T*)bias, (float*)q_out, (T*)kcache, (T*)vcache,
                             (const int*)tok_seq, (const int*)tok_pos, (const int*)tables, max_blocks, block_size, Hq,
                             G, d, dv, eps, normalize)));
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}

/* As sxb_qk_norm_append for projections that pass a short causal filter over time first (conv_w `dtype` [C, taps] with
 * C = Hq*d + G*d + G*dv, last tap = current token, or null; carried inputs state `dtype` [slots, taps-1, C], to be moved
 * on with sxb_conv_state_update afterwards), with a norm weight of d entries shared by the heads (q_w / k_w, `dtype`, or
 * null) and a query temperature 1 + temp_coef * ln(floor((pos + 1) / temp_every) + 1). */
SXB_API int sxb_qkv_filter_norm_append(const void* qkv, long long ld, const void* conv_w, const void* state,
                                       const void* seq_info, const void* q_w, const void* k_w, void* q_out,
                                       void* kcache, void* vcache, const void* tok_seq, const void* tok_pos,
                                       const void* tables, int n_tokens, int max_blocks, int block_size, int Hq, int G,
                                       int d, int dv, int taps, float eps, int normalize, float temp_coef,
                                       int temp_every, int dtype, void* stream) {
  if (n_tokens <= 0) return SXB_OK;
  if (d > 256 || dv > 256 || taps < 1 || taps > kMaxTaps || temp_every < 1) return SXB_ERR_UNSUPPORTED;
  if (conv_w != nullptr && taps > 1 && state == nullptr) return SXB_ERR_BAD_ARG;
  const int widest = std::max(d, dv);
  const int vecw = widest <= 32 ? 1 : (widest <= 64 ? 2 : (widest <= 128 ? 4 : 8));
  // one access per lane needs every head to start on a multiple of the lane's channels, in the rows and the caches
  const int vec_ok = d % vecw == 0 && dv % vecw == 0 && ld % vecw == 0 &&
                     ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(state) |
                       reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(kcache) |
                       reinterpret_cast<uintptr_t>(vcache)) & 31) == 0;
  // prompt batches: a warp walks 8 rows (filters of 2 to 4 taps); few rows: one row per warp spreads them over more CTAs
  const int ktaps = (conv_w != nullptr && taps >= 2 && taps <= 4) ? taps : 0;
  const int rpw = (ktaps > 0 && n_tokens >= 1024) ? 8 : 1;
  const dim3 grid((n_tokens + rpw - 1) / rpw, (Hq + 2 * G + 3) / 4);
  if (conv_w == nullptr) taps = 1;
#define FILTER_APPEND_T(VEC, TAPS)                                                                                     \
  SEQMIX_DISPATCH(dtype, (qkv_filter_norm_append_kernel<T, VEC, TAPS><<<grid, 128, 0, (cudaStream_t)stream>>>(         \
                             (const T*)qkv, ld, (const T*)conv_w, (const T*)state, (const int*)seq_info, (const T*)q_w, \
                             (const T*)k_w, (float*)q_out, (T*)kcache, (T*)vcache, (const int*)tok_seq,                \
                             (const int*)tok_pos, (const int*)tables, max_blocks, block_size, Hq, G, d, dv, taps, eps, \
                             normalize, temp_coef, temp_every, vec_ok, n_tokens, rpw)))
#define FILTER_APPEND(VEC)                 \
  do {                                     \
    if (ktaps == 2) FILTER_APPEND_T(VEC, 2);      \
    else if (ktaps == 3) FILTER_APPEND_T(VEC, 3); \
    else if (ktaps == 4) FILTER_APPEND_T(VEC, 4); \
    else FILTER_APPEND_T(VEC, 0);                 \
  } while (0)
  if (vecw == 1) FILTER_APPEND(1);
  else if (vecw == 2) FILTER_APPEND(2);
  else if (vecw == 4) FILTER_APPEND(4);
  else FILTER_APPEND(8);
#undef FILTER_APPEND_T
#undef FILTER_APPEND
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}

/* Attention of every token over the cached keys lo..pos of its sequence, scores and weights in fp32.  lo = start of the
 * token's chunk of `chunk` positions (chunk > 0), else pos - window + 1 clamped at 0 (window > 0), else 0.  sink (fp32
 * [Hq] or null) adds exp(sink[h]) to the denominator.  Key rows sit at kcache + slot * k_pitch + g * d and value rows at
 * vcache + slot * v_pitch + g * dv (pitches in elements; 0 = packed [pages, block_size, G, d|dv]), so values may be a
 * column range of the key rows.  out `dtype` [n_tokens, Hq * dv] (the caches have the same type).  dist_bias (fp32
 * [Hq, bias_len] or null) is added to the scaled score of a key at distance n = query position - key position:
 * dist_bias[h, min(n, bias_len - 1)].  gate (`dtype` rows of pitch gate_ld with Hq * dv channels, or null): the output is
 * multiplied by sigmoid(gate).  One CTA per (token, head group). */
SXB_API int sxb_sink_attention(const void* q, const void* kcache, const void* vcache, const void* sink, void* out,
                               const void* tok_seq, const void* tok_pos, const void* tables, int n_tokens,
                               int max_blocks, int block_size, int Hq, int G, int d, int dv, float scale, int chunk,
                               int window, int k_pitch, int v_pitch, const void* dist_bias, int bias_len,
                               const void* gate, long long gate_ld, int dtype, void* stream) {
  if (n_tokens <= 0) return SXB_OK;
  if (dv > 32 * kMaxVPerLane || Hq % G || (dist_bias != nullptr && bias_len < 1)) return SXB_ERR_UNSUPPORTED;
  if (k_pitch <= 0) k_pitch = G * d;
  if (v_pitch <= 0) v_pitch = G * dv;
  const int rc = attention_rows(dtype, dim3(n_tokens, 1), q, kcache, vcache, sink, out, tok_seq, tok_pos, tables,
                                max_blocks, block_size, Hq, G, d, dv, scale, chunk, window, k_pitch, v_pitch, nullptr,
                                dist_bias, bias_len, gate, gate_ld, (cudaStream_t)stream);
  if (rc != SXB_OK) return rc;
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}


// ------------------------------------------------------------------------------------------------ token side input
// g[t, c] = gelu_tanh(gx[t, c]) * table[ids[t], col0 + c] for c < dim, 0 for dim <= c < out_w.
template <typename T>
__global__ void __launch_bounds__(256)
side_gate_kernel(const T* __restrict__ gx, long long ld, const T* __restrict__ table, long long table_ld,
                 const int* __restrict__ ids, T* __restrict__ out, long long total, int dim, int out_w, int col0) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / out_w;
  const int c = (int)(i % out_w);
  float g = 0.f;
  if (c < dim) {
    const float z = to_f32<T>(gx[t * ld + c]);
    const float a = 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    g = a * to_f32<T>(table[(long long)ids[t] * table_ld + col0 + c]);
  }
  out[i] = from_f32<T>(g);
}

// x <- cap * tanh(x * scale / cap) (cap > 0), or x * scale; fp32 in place.
__global__ void __launch_bounds__(256)
scale_softcap_kernel(float* __restrict__ x, long long total, float scale, float cap) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const float z = x[i] * scale;
  x[i] = cap > 0.f ? cap * tanhf(z / cap) : z;
}

// acc[t, c] += sigmoid(gate[t]) * y[t, c]: gate fp32 with a row pitch, acc and y in the activation type.
template <typename T>
__global__ void __launch_bounds__(256)
row_gate_add_kernel(T* __restrict__ acc, const T* __restrict__ y, const float* __restrict__ gate, long long gate_ld,
                    long long total, int width) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const float g = sigmoid_f(gate[(i / width) * gate_ld]);
  acc[i] = from_f32<T>(to_f32<T>(acc[i]) + g * to_f32<T>(y[i]));
}

// The same with 16-byte accesses: a thread takes 16 / sizeof(T) consecutive channels of one row.
template <typename T>
__global__ void __launch_bounds__(256)
row_gate_add_vec_kernel(T* __restrict__ acc, const T* __restrict__ y, const float* __restrict__ gate, long long gate_ld,
                        long long n_vec, int vec_per_row) {
  constexpr int PER = 16 / (int)sizeof(T);
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_vec) return;
  const float g = sigmoid_f(gate[(i / vec_per_row) * gate_ld]);
  Pack<T, PER> a = reinterpret_cast<Pack<T, PER>*>(acc)[i];
  const Pack<T, PER> b = reinterpret_cast<const Pack<T, PER>*>(y)[i];
#pragma unroll
  for (int e = 0; e < PER; ++e) a.v[e] = from_f32<T>(to_f32<T>(a.v[e]) + g * to_f32<T>(b.v[e]));
  reinterpret_cast<Pack<T, PER>*>(acc)[i] = a;
}

// Router product in 32-bit: logits[t, r] = bias[r] + sum_c x[t, c] * w[r, c] with x in the activation type (its values
// taken as they are: no 32-bit copy of the rows is made) and w, bias, logits fp32.  CTAs of eight warps; WPT warps share
// the columns of one token (prompt batches: one warp per token, eight tokens per CTA, the weights of the few router
// rows are re-read from L1 by the other warps; few rows: the eight warps of a CTA split one token's columns and add
// their parts in shared memory).  A lane takes 4 consecutive columns at a time.
constexpr int kRouterRows = 16;

template <typename T, int WPT>
__global__ void __launch_bounds__(256)
router_logits_kernel(const T* __restrict__ x, long long ld, const float* __restrict__ w, const float* __restrict__ bias,
                     float* __restrict__ out, int n_tokens, int width, int R) {
  __shared__ float part_sum[8][kRouterRows];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int part = warp % WPT;
  const int t = blockIdx.x * (8 / WPT) + warp / WPT;
  const bool active = t < n_tokens;
  float acc[kRouterRows];
#pragma unroll
  for (int r = 0; r < kRouterRows; ++r) acc[r] = 0.f;
  if (active) {
    const T* row = x + (long long)t * ld;
    for (int c = (part * 32 + lane) * 4; c < width; c += 128 * WPT) {
      float xv[4];
      load_pack<T, 4>(row + c, xv, true, 4);
#pragma unroll
      for (int r = 0; r < kRouterRows; ++r) {
        if (r < R) {
          const float4 wv = *reinterpret_cast<const float4*>(w + (long long)r * width + c);
          acc[r] += (xv[0] * wv.x + xv[1] * wv.y) + (xv[2] * wv.z + xv[3] * wv.w);
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < kRouterRows; ++r) {
    if (r < R) {
      const float v = warp_sum(acc[r]);
      if (WPT == 1) {
        if (active && lane == 0) out[(long long)t * R + r] = v + (bias ? bias[r] : 0.f);
      } else if (lane == 0) {
        part_sum[warp][r] = v;
      }
    }
  }
  if (WPT > 1) {
    __syncthreads();
    if (active && part == 0 && lane < R) {
      float v = bias ? bias[lane] : 0.f;
      for (int p = 0; p < WPT; ++p) v += part_sum[warp + p][lane];
      out[(long long)t * R + lane] = v;
    }
  }
}

template <typename T, int NV>
static int launch_attention_tiles(const void* q, const void* kcache, const void* vcache, const void* sink, void* out,
                                  const void* atoms, int n_long, const void* tables, int max_blocks, int block_size,
                                  int Hq, int G, int d, int dv, float scale, int chunk, int window, int kpitch,
                                  int vpitch, const void* dist_bias, int bias_len, const void* gate,
                                  long long gate_ld, cudaStream_t s) {
  const size_t smem = (size_t)(kBQ * (d + 4) + std::max(kBK * (d + 4), kBQ * (kBK + 4)) + kBK * NV * 64) * sizeof(float);
  cudaError_t e = cudaFuncSetAttribute(sink_attention_tile_kernel<T, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem);
  if (e != cudaSuccess) return (int)e;
  sink_attention_tile_kernel<T, NV><<<dim3(2 * n_long, Hq), 256, smem, s>>>(
      (const float*)q, (const T*)kcache, (const T*)vcache, (const float*)sink, (T*)out, (const int*)atoms,
      (const int*)tables, max_blocks, block_size, Hq, G, d, dv, scale, chunk, window, kpitch, vpitch,
      (const float*)dist_bias, bias_len, (const T*)gate, gate_ld);
  return SXB_OK;
}

/* The same attention scheduled by attention atoms int32 [n_atoms, 6] = (sequence, first row, queries, first position,
 * -, -), longest first: the first n_long atoms (more than 16 queries, at most 128) run the tiled kernel, 64 queries per
 * CTA; the others one warp per (query, head).  Needs d, dv and both pitches multiples of 4, d and dv at most 256. */
SXB_API int sxb_sink_attention_atoms(const void* q, const void* kcache, const void* vcache, const void* sink, void* out,
                                     const void* atoms, int n_atoms, int n_long, const void* tables, int max_blocks,
                                     int block_size, int Hq, int G, int d, int dv, float scale, int chunk, int window,
                                     int k_pitch, int v_pitch, const void* dist_bias, int bias_len, const void* gate,
                                     long long gate_ld, int dtype, void* stream) {
  if (n_atoms <= 0) return SXB_OK;
  if (dist_bias != nullptr && bias_len < 1) return SXB_ERR_UNSUPPORTED;
  if (k_pitch <= 0) k_pitch = G * d;
  if (v_pitch <= 0) v_pitch = G * dv;
  if (d % 4 || dv % 4 || k_pitch % 4 || v_pitch % 4 || d > 256 || dv > 256 || Hq % G || n_long < 0 || n_long > n_atoms)
    return SXB_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  if (n_long > 0) {
    const int nv = (dv + 63) / 64;
    int rc = SXB_OK;
#define TILES(NV)                                                                                                     \
  SEQMIX_DISPATCH(dtype, (rc = launch_attention_tiles<T, NV>(q, kcache, vcache, sink, out, atoms, n_long, tables,      \
                                                              max_blocks, block_size, Hq, G, d, dv, scale, chunk,      \
                                                              window, k_pitch, v_pitch, dist_bias, bias_len, gate,     \
                                                              gate_ld, s)))
    if (nv == 1) TILES(1);
    else if (nv == 2) TILES(2);
    else if (nv == 3) TILES(3);
    else TILES(4);
#undef TILES
    if (rc != SXB_OK) return rc;
    SXB_CHECK_LAUNCH();
  }
  if (n_atoms > n_long) {
    const int rc = attention_rows(dtype, dim3((n_atoms - n_long) * kShortAtom, 1), q, kcache, vcache, sink, out, nullptr,
                                  nullptr, tables, max_blocks, block_size, Hq, G, d, dv, scale, chunk, window, k_pitch,
                                  v_pitch, (const int*)atoms + 6 * n_long, dist_bias, bias_len, gate, gate_ld, s);
    if (rc != SXB_OK) return rc;
    SXB_CHECK_LAUNCH();
  }
  return SXB_OK;
}

/* Short causal filter + SiLU over C channels of x [n_tokens, ld] (`dtype`), w [C, taps] (last tap = current token),
 * bias [C] or null, carried inputs state [slots, taps-1, C]; out fp32 [n_tokens, C].  seq_info int32 [n_seqs, 4] =
 * {first row, rows, seen tokens, slot}. */
SXB_API int sxb_conv_silu(const void* x, long long ld, const void* w, const void* bias, const void* state,
                          const void* seq_info, const void* tok_seq, void* out, int n_tokens, int C, int taps,
                          int dtype, void* stream) {
  if (n_tokens <= 0) return SXB_OK;
  if (taps < 1 || taps > kMaxTaps) return SXB_ERR_UNSUPPORTED;
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(state) |
                         reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  // few rows (decode batches): the one-thread-per-element kernel spreads them over more CTAs
  if (n_tokens >= 128 && taps >= 2 && taps <= 4 && C % 8 == 0 && ld % 8 == 0 && aligned) {
    dim3 vgrid((n_tokens + kConvRows - 1) / kConvRows, (C / 8 + 127) / 128);
#define CONV_VEC(TAPS)                                                                                             \
  SEQMIX_DISPATCH(dtype, (conv_silu_vec_kernel<T, TAPS><<<vgrid, 128, 0, (cudaStream_t)stream>>>(                  \
                             (const T*)x, ld, (const T*)w, (const T*)bias, (const T*)state, (const int*)seq_info,  \
                             (const int*)tok_seq, (float*)out, C, n_tokens)))
    if (taps == 2) CONV_VEC(2);
    else if (taps == 3) CONV_VEC(3);
    else CONV_VEC(4);
#undef CONV_VEC
    SXB_CHECK_LAUNCH();
    return SXB_OK;
  }
  dim3 grid(n_tokens, (C + 1023) / 1024);
  SEQMIX_DISPATCH(dtype, (conv_silu_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>(
                             (const T*)x, ld, (const T*)w, (const T*)bias, (const T*)state, (const int*)seq_info,
                             (const int*)tok_seq, (float*)out, C, taps)));
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}

/* Run after sxb_conv_silu on the same batch: every sequence's slot keeps its last taps-1 inputs. */
SXB_API int sxb_conv_state_update(const void* x, long long ld, void* state, const void* seq_info, int n_seqs, int C,
                                  int taps, int dtype, void* stream) {
  if (n_seqs <= 0 || taps <= 1) return SXB_OK;
  if (taps > kMaxTaps) return SXB_ERR_UNSUPPORTED;
  dim3 grid(n_seqs, (C + 255) / 256);
  SEQMIX_DISPATCH(dtype, (conv_state_update_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>(
                             (const T*)x, ld, (T*)state, (const int*)seq_info, C, taps)));
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}

/* In place on fp32 rows x [n_tokens, ld]: heads of `dim` channels starting at col0 become x * mult / sqrt(sum x^2 + eps). */
SXB_API int sxb_unit_norm_heads(void* x, long long ld, int col0, int n_heads, int dim, float mult, float eps,
                                int n_tokens, void* stream) {
  if (n_tokens <= 0 || n_heads <= 0) return SXB_OK;
  const int total = n_tokens * n_heads;
  unit_norm_heads_kernel<<<(total + 3) / 4, 128, 0, (cudaStream_t)stream>>>((float*)x, ld, col0, n_heads, dim, mult, eps,
                                                                           n_tokens);
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}

/* decay, beta fp32 [n_tokens, H] from raw projections (`dtype`, row pitch ld, H channels each), A_log / dt_bias fp32 [H].
 * mode 0: beta = sigmoid(b_raw), decay = exp(-exp(A_log) softplus(a_raw + dt_bias)).
 * mode 1: beta = softplus(a_raw + dt_bias) (b_raw unused), decay = exp(-exp(A_log) beta). */
SXB_API int sxb_recurrence_gates(const void* a_raw, const void* b_raw, long long ld, const void* A_log,
                                 const void* dt_bias, void* decay, void* beta, int H, int n_tokens, int mode, int dtype,
                                 void* stream) {
  if (n_tokens <= 0) return SXB_OK;
  const int total = n_tokens * H;
  SEQMIX_DISPATCH(dtype, (recurrence_gates_kernel<T><<<(total + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
                             (const T*)a_raw, (const T*)b_raw, ld, (const float*)A_log, (const float*)dt_bias,
                             (float*)decay, (float*)beta, H, n_tokens, mode)));
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}

/* decay_channels != 0: decay fp32 [rows, H * n] holds one factor per (head, key channel) pair (it scales the state entries of that key channel).
 * Per sequence and head, rows in order:  S <- decay S;  u = beta (v - [delta] S^T k);  S <- S + k u^T;
 * o = S^T q (+ skip[h] v).  kvec / qvec fp32 [rows, ldkq] hold G heads of n channels, val fp32 [rows, ldv] H heads of dv,
 * decay / beta fp32 [rows, H], state fp32 [slots, H, dv, n] (taken as zero when the sequence has seen no token), out fp32
 * [rows, H * dv]. */
SXB_API int sxb_linear_recurrence(const void* kvec, const void* qvec, long long ldkq, const void* val, long long ldv,
                                  const void* decay, const void* beta, const void* skip, void* state, void* out,
                                  const void* seq_info, int n_seqs, int H, int G, int n, int dv, int delta,
                                  int decay_channels, void* stream) {
  if (n_seqs <= 0) return SXB_OK;
  if (n > 256 || H % G) return SXB_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
#define LAUNCH_REC(R, D, LPC, CH)                                                                                   \
  do {                                                                                                              \
    constexpr int cols = kRecThreads / LPC;                                                                         \
    const size_t smem = (size_t)2 * ((CH ? 3 : 2) * kTB * (R * LPC) + kTB * cols + 2 * kTB) * sizeof(float);        \
    if (smem > 48 * 1024)                                                                                           \
      cudaFuncSetAttribute(linear_recurrence_kernel<R, D, LPC, CH>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                           (int)smem);                                                                              \
    linear_recurrence_kernel<R, D, LPC, CH><<<dim3((dv + cols - 1) / cols, H, n_seqs), kRecThreads, smem, s>>>(     \
        (const float*)kvec, (const float*)qvec, ldkq, (const float*)val, ldv, (const float*)decay,                  \
        (const float*)beta, (const float*)skip, (float*)state, (float*)out, (const int*)seq_info, H, G, n, dv);     \
  } while (0)
#define LAUNCH_REC_N(D, CH)                                  \
  if (n <= 32) LAUNCH_REC(4, D, 8, CH);                      \
  else if (n <= 64) LAUNCH_REC(8, D, 8, CH);                 \
  else if (n <= 128) LAUNCH_REC(16, D, 8, CH);               \
  else LAUNCH_REC(32, D, 8, CH)
  if (decay_channels) {
    if (delta) { LAUNCH_REC_N(true, true); } else { LAUNCH_REC_N(false, true); }
  } else {
    if (delta) { LAUNCH_REC_N(true, false); } else { LAUNCH_REC_N(false, false); }
  }
#undef LAUNCH_REC_N
#undef LAUNCH_REC
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}

/* RMS norm over groups of gs channels of y fp32 [n_tokens, C] with a SiLU gate (`dtype` rows of pitch ldg) and a weight
 * of wlen entries that repeats along the row.  gate_first bit 0: norm(y silu(gate)) w; else norm(y) w silu(gate); bit 1:
 * sigmoid(gate) in place of silu(gate). */
SXB_API int sxb_group_norm_gate(const void* y, const void* gate, long long ldg, const void* w, int wlen, void* out,
                                int n_tokens, int C, int gs, float eps, int gate_first, int dtype, void* stream) {
  if (n_tokens <= 0) return SXB_OK;
  if (gs <= 0 || C % gs) return SXB_ERR_BAD_ARG;
  dim3 grid(n_tokens, C / gs);
  SEQMIX_DISPATCH(dtype, (group_norm_gate_kernel<T><<<grid, 128, 0, (cudaStream_t)stream>>>(
                             (const float*)y, (const T*)gate, ldg, (const T*)w, wlen, (T*)out, C, gs, eps, gate_first)));
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}

/* out [rows, F] = act(in[:, :F]) * in[:, F:] for rows of any width; act: 0 identity, 1 relu, 2 gelu (tanh form), 3 silu,
 * 5 clamped: a = min(gate, L), b = max(-L, min(up, L)), out = a sigmoid(1.702 a) (1 + b). */
SXB_API int sxb_gated_act_rows(const void* in, void* out, long long rows, int F, int act, int dtype, float limit,
                               void* stream) {
  const long long total = rows * F;
  if (total <= 0) return SXB_OK;
  const int per = dtype == 0 ? 4 : 8;
  if (F % per == 0 && ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0 &&
      (dtype == 0 || dtype == 2)) {
    const long long nv = total / per;
    if (dtype == 0)
      gated_act_rows_vec_kernel<float, 4><<<(unsigned)((nv + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
          (const float*)in, (float*)out, nv, F / 4, act, limit);
    else
      gated_act_rows_vec_kernel<__nv_bfloat16, 8><<<(unsigned)((nv + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
          (const __nv_bfloat16*)in, (__nv_bfloat16*)out, nv, F / 8, act, limit);
    SXB_CHECK_LAUNCH();
    return SXB_OK;
  }
  SEQMIX_DISPATCH(dtype, (gated_act_rows_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
                             (const T*)in, (T*)out, total, F, act, limit)));
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}

/* out `dtype` [n_tokens, C] = x + causal filter of x over time per channel: x fp32 [n_tokens, C], w `dtype` [C, taps]
 * (last tap = current token), carried inputs state fp32 [slots, taps-1, C] (update them with sxb_conv_state_update,
 * dtype fp32, afterwards). */
SXB_API int sxb_conv_residual(const void* x, const void* w, const void* state, const void* seq_info,
                              const void* tok_seq, void* out, int n_tokens, int C, int taps, int dtype, void* stream) {
  if (n_tokens <= 0) return SXB_OK;
  if (taps < 1) return SXB_ERR_BAD_ARG;
  dim3 grid(n_tokens, (C + 1023) / 1024);
  SEQMIX_DISPATCH(dtype, (conv_residual_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>(
                             (const float*)x, (const T*)w, (const float*)state, (const int*)seq_info,
                             (const int*)tok_seq, (T*)out, C, taps)));
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}

/* Per row: v = x_in + ls (.) (y / rms(y) * gain[0]) -> x_out (fp32, may alias x_in); y `dtype`, gain / ls fp32.  With
 * mix_out (fp32): mix_out = sum_{j < n_prev} mixw[j] * (stack + j * stack_stride)[row] + mixw[n_prev] * v. */
SXB_API int sxb_post_norm_mix(const void* x_in, const void* y, const void* gain, const void* ls, void* x_out,
                              const void* stack, long long stack_stride, int n_prev, const void* mixw, void* mix_out,
                              long long rows, int width, float eps, int dtype, void* stream) {
  if (rows <= 0) return SXB_OK;
  if (mix_out != nullptr && (mixw == nullptr || (n_prev > 0 && stack == nullptr))) return SXB_ERR_BAD_ARG;
  SEQMIX_DISPATCH(dtype, (post_norm_mix_kernel<T><<<(unsigned)rows, 256, 0, (cudaStream_t)stream>>>(
                             (const float*)x_in, (const T*)y, (const float*)gain, (const float*)ls, (float*)x_out,
                             (const float*)stack, stack_stride, n_prev, (const float*)mixw, (float*)mix_out, width,
                             eps)));
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}

/* out `dtype` [n_rows, width] = x[rows[i]] / rms * gain[0]; x fp32, rows int32 or null (all rows in order). */
SXB_API int sxb_rms_scale_rows(const void* x, const void* rows, const void* gain, void* out, int n_rows, int width,
                               float eps, int dtype, void* stream) {
  if (n_rows <= 0) return SXB_OK;
  SEQMIX_DISPATCH(dtype, (rms_scale_rows_kernel<T><<<n_rows, 256, 0, (cudaStream_t)stream>>>(
                             (const float*)x, (const int*)rows, (const float*)gain, (T*)out, width, eps)));
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}

/* out `dtype` [n_tokens, n] = x[:, :n] / rms * w; x rows of pitch ld. */
SXB_API int sxb_rms_norm_slice(const void* x, long long ld, const void* w, void* out, int n_tokens, int n, float eps,
                               int dtype, void* stream) {
  if (n_tokens <= 0) return SXB_OK;
  SEQMIX_DISPATCH(dtype, (rms_norm_slice_kernel<T><<<n_tokens, 128, 0, (cudaStream_t)stream>>>(
                             (const T*)x, ld, (const T*)w, (T*)out, n, eps)));
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}

/* out = act(in + bias) over rows of F channels; act: 0 identity, 1 relu, 2 gelu (tanh form), 3 silu, 4 relu squared. */
SXB_API int sxb_bias_act_rows(const void* in, const void* bias, void* out, long long rows, int F, int act, int dtype,
                              void* stream) {
  const long long total = rows * F;
  if (total <= 0) return SXB_OK;
  const int per = dtype == 0 ? 4 : 8;
  if (F % per == 0 && ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out) |
                        reinterpret_cast<uintptr_t>(bias)) & 15) == 0) {
    const long long nv = total / per;
    SEQMIX_DISPATCH(dtype, (bias_act_rows_vec_kernel<T><<<(unsigned)((nv + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
                               (const T*)in, (const T*)bias, (T*)out, nv, F, act)));
    SXB_CHECK_LAUNCH();
    return SXB_OK;
  }
  SEQMIX_DISPATCH(dtype, (bias_act_rows_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
                             (const T*)in, (const T*)bias, (T*)out, total, F, act)));
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}

/* Latent attention, per token: cache[page, offset] = [kv[:r] / rms * w_norm | rope(kv[r : r+rot])] (`dtype`
 * [pages, block_size, r + rot]); q_out fp32 [n_tokens, H, r + rot] = [qabs[t, h] | rope(qfull[t, h, dim : dim+rot])].
 * qfull rows of pitch ldq hold H heads of dim + rot; qabs element (t, h, c) at t * qa_tok + h * qa_head + c; kv rows of
 * pitch ldkv; inv_freq fp32 [rot_dims / 2]; amp multiplies the turned channels of q and k. */
SXB_API int sxb_latent_qk_prepare(const void* qfull, long long ldq, const void* qabs, long long qa_tok,
                                  long long qa_head, const void* kv, long long ldkv, const void* w_norm,
                                  const void* inv_freq, void* q_out, void* cache, const void* tok_seq,
                                  const void* tok_pos, const void* tables, int n_tokens, int max_blocks, int block_size,
                                  int H, int dim, int rot, int r, int rot_dims, float eps, int dtype, float amp,
                                  void* stream) {
  if (n_tokens <= 0) return SXB_OK;
  if (rot_dims > rot || (rot_dims & 1)) return SXB_ERR_BAD_ARG;
  SEQMIX_DISPATCH(dtype, (latent_qk_prepare_kernel<T><<<n_tokens, 128, 0, (cudaStream_t)stream>>>(
                             (const T*)qfull, ldq, (const T*)qabs, qa_tok, qa_head, (const T*)kv, ldkv,
                             (const T*)w_norm, (const float*)inv_freq, (float*)q_out, (T*)cache, (const int*)tok_seq,
                             (const int*)tok_pos, (const int*)tables, max_blocks, block_size, H, dim, rot, r, rot_dims,
                             eps, amp)));
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}

/* buf fp32 [n_tokens, 2 H n + H (dv + 1)] = [q * qscale | k | per head (v, 1)] from projection rows (pitch ld) that
 * start with q (H n) | k (H n) | v (H dv). */
SXB_API int sxb_mlstm_prepare(const void* proj, long long ld, void* buf, int n_tokens, int H, int n, int dv,
                              float qscale, int dtype, void* stream) {
  if (n_tokens <= 0) return SXB_OK;
  SEQMIX_DISPATCH(dtype, (mlstm_prepare_kernel<T><<<n_tokens, 256, 0, (cudaStream_t)stream>>>(
                             (const T*)proj, ld, (float*)buf, H, n, dv, qscale)));
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}

/* Gates of the matrix-memory LSTM: raw_i / raw_f (`dtype`, pitch ld, H channels), biases fp32 [H]; i = cap tanh((raw_i +
 * b_i) / cap), f = logsigmoid(cap tanh((raw_f + b_f) / cap)); m_t = max(f_t + m_(t-1), i_t) from mstate fp32 [slots, H]
 * (0 for a sequence that has seen no token; written back).  decay = exp(f + m_(t-1) - m_t), beta = exp(i - m_t), mt = m_t,
 * all fp32 [n_tokens, H]. */
SXB_API int sxb_mlstm_gate_scan(const void* raw_i, const void* raw_f, long long ld, const void* bias_i,
                                const void* bias_f, float cap, void* mstate, void* decay, void* beta, void* mt,
                                const void* seq_info, int n_seqs, int n_tokens, int H, int dtype, void* stream) {
  if (n_seqs <= 0) return SXB_OK;
  // threads per (sequence, head): the mean number of rows of a sequence, in whole warps
  const int mean_rows = (n_tokens + n_seqs - 1) / n_seqs;
  const int threads = std::min(kScanThreads, std::max(32, (mean_rows + 31) / 32 * 32));
  SEQMIX_DISPATCH(dtype, (mlstm_gate_scan_kernel<T><<<dim3(n_seqs, H), threads, 0, (cudaStream_t)stream>>>(
                             (const T*)raw_i, (const T*)raw_f, ld, (const float*)bias_i, (const float*)bias_f, cap,
                             (float*)mstate, (float*)decay, (float*)beta, (float*)mt, (const int*)seq_info, H)));
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}

/* out `dtype` [n_tokens, H dv]: per head unit_rms(o[:dv] / (max(|o[dv]|, exp(-mt)) + 1e-6)) * w * sigmoid(gate); o fp32
 * [n_tokens, H (dv + 1)], gate `dtype` rows of pitch ldg, w `dtype` [H dv]. */
SXB_API int sxb_mlstm_output(const void* o, const void* mt, const void* gate, long long ldg, const void* w, void* out,
                             int n_tokens, int H, int dv, float eps, int dtype, void* stream) {
  if (n_tokens <= 0) return SXB_OK;
  const int total = n_tokens * H;
  SEQMIX_DISPATCH(dtype, (mlstm_output_kernel<T><<<(total + 3) / 4, 128, 0, (cudaStream_t)stream>>>(
                             (const float*)o, (const float*)mt, (const T*)gate, ldg, (const T*)w, (T*)out, n_tokens, H,
                             dv, eps)));
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}

/* Gate of a per-layer token input: out `dtype` [n_tokens, out_w] = gelu_tanh(gx[:, :dim]) * table[ids, col0 : col0 + dim],
 * zero in the columns dim .. out_w - 1 (padding up to the next product's alignment).  gx rows of pitch ld, table rows of
 * pitch table_ld. */
SXB_API int sxb_side_gate(const void* gx, long long ld, const void* table, long long table_ld, const void* ids, void* out,
                          int n_tokens, int dim, int out_w, int col0, int dtype, void* stream) {
  const long long total = (long long)n_tokens * out_w;
  if (total <= 0) return SXB_OK;
  if (dim > out_w) return SXB_ERR_BAD_ARG;
  SEQMIX_DISPATCH(dtype, (side_gate_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
                             (const T*)gx, ld, (const T*)table, table_ld, (const int*)ids, (T*)out, total, dim, out_w,
                             col0)));
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}

/* In place on fp32 x [total]: x * scale, then cap * tanh(. / cap) when cap > 0. */
SXB_API int sxb_scale_softcap(void* x, long long total, float scale, float cap, void* stream) {
  if (total <= 0) return SXB_OK;
  scale_softcap_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>((float*)x, total, scale, cap);
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}

/* acc `dtype` [rows, width] += sigmoid(gate[row]) * y; gate fp32, one number per row at pitch gate_ld. */
SXB_API int sxb_row_gate_add(void* acc, const void* y, const void* gate, long long gate_ld, long long rows, int width,
                             int dtype, void* stream) {
  const long long total = rows * width;
  if (total <= 0) return SXB_OK;
  const int per = dtype == 0 ? 4 : 8;
  if (width % per == 0 && ((reinterpret_cast<uintptr_t>(acc) | reinterpret_cast<uintptr_t>(y)) & 15) == 0) {
    const long long nv = total / per;
    SEQMIX_DISPATCH(dtype, (row_gate_add_vec_kernel<T><<<(unsigned)((nv + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
                               (T*)acc, (const T*)y, (const float*)gate, gate_ld, nv, width / per)));
    SXB_CHECK_LAUNCH();
    return SXB_OK;
  }
  SEQMIX_DISPATCH(dtype, (row_gate_add_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
                             (T*)acc, (const T*)y, (const float*)gate, gate_ld, total, width)));
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}

/* Router logits in 32-bit: out fp32 [n_tokens, R] = x[:, :width] w^T + bias; x `dtype` rows of pitch ld, w fp32 [R, width],
 * bias fp32 [R] or null.  Up to 16 router rows, width and pitch multiples of 4, x and w 16-byte aligned. */
SXB_API int sxb_router_logits(const void* x, long long ld, const void* w, const void* bias, void* out, int n_tokens,
                              int width, int R, int dtype, void* stream) {
  if (n_tokens <= 0 || R <= 0) return SXB_OK;
  if (R > kRouterRows || width % 4 || ld % 4 ||
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) != 0)
    return SXB_ERR_UNSUPPORTED;
  if (n_tokens >= 1024) {
    SEQMIX_DISPATCH(dtype, (router_logits_kernel<T, 1><<<(n_tokens + 7) / 8, 256, 0, (cudaStream_t)stream>>>(
                               (const T*)x, ld, (const float*)w, (const float*)bias, (float*)out, n_tokens, width, R)));
  } else {
    SEQMIX_DISPATCH(dtype, (router_logits_kernel<T, 8><<<n_tokens, 256, 0, (cudaStream_t)stream>>>(
                               (const T*)x, ld, (const float*)w, (const float*)bias, (float*)out, n_tokens, width, R)));
  }
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}

// ------------------------------------------------------------------------------------------------ gates and activations
namespace sxb {
namespace seqmix {

// x[t, c] *= sigmoid(gate[t, c / group]) in place: group 1 is one gate per channel, group = head size one per head.
template <typename T>
__global__ void __launch_bounds__(256)
sigmoid_gate_rows_kernel(T* __restrict__ x, const T* __restrict__ gate, long long ldg, long long total, int width,
                         int group) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / width;
  const int c = (int)(i % width);
  x[i] = from_f32<T>(to_f32<T>(x[i]) * sigmoid_f(to_f32<T>(gate[t * ldg + c / group])));
}

// The same with 8 (bf16) or 4 (fp32) consecutive channels per thread: 16-byte accesses of x, and of the gate when it is
// per channel; a per-head gate is read once per thread (group is then a multiple of the vector length).
template <typename T, int VEC>
__global__ void __launch_bounds__(256)
sigmoid_gate_rows_vec_kernel(T* __restrict__ x, const T* __restrict__ gate, long long ldg, long long nvec, int wvec,
                             int group) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nvec) return;
  const long long t = i / wvec;
  const int c = (int)(i % wvec) * VEC;
  struct alignas(16) Pack { T v[VEC]; };
  Pack xv = *reinterpret_cast<const Pack*>(x + i * VEC);
  if (group == 1) {
    const Pack gv = *reinterpret_cast<const Pack*>(gate + t * ldg + c);
#pragma unroll
    for (int j = 0; j < VEC; ++j) xv.v[j] = from_f32<T>(to_f32<T>(xv.v[j]) * sigmoid_f(to_f32<T>(gv.v[j])));
  } else {
    const float s = sigmoid_f(to_f32<T>(gate[t * ldg + c / group]));
#pragma unroll
    for (int j = 0; j < VEC; ++j) xv.v[j] = from_f32<T>(to_f32<T>(xv.v[j]) * s);
  }
  *reinterpret_cast<Pack*>(x + i * VEC) = xv;
}

// Three-power normalised activation, one CTA per row of F channels:
//   z = x + bias;  out = p1 z / rms(z) + p2 z^2 / rms(z^2) + p3 z^3 / rms(z^3) + p0,   rms(u) = sqrt(mean(u^2) + eps)
// coef fp32 [4] = (p1, p2, p3, p0).  The three sums of squares (z^2, z^4, z^6) come from one pass in 32-bit.
template <typename T>
__global__ void __launch_bounds__(256)
power_norm_act_kernel(const T* __restrict__ x, const T* __restrict__ bias, const float* __restrict__ coef,
                      T* __restrict__ out, int F, float eps) {
  __shared__ float red[32];
  const long long base = (long long)blockIdx.x * F;
  float s1 = 0.f, s2 = 0.f, s3 = 0.f;
  for (int c = threadIdx.x; c < F; c += blockDim.x) {
    const float z = to_f32<T>(x[base + c]) + (bias ? to_f32<T>(bias[c]) : 0.f);
    const float z2 = z * z;
    s1 += z2, s2 += z2 * z2, s3 += z2 * z2 * z2;
  }
  s1 = block_sum(s1, red);
  __syncthreads();
  s2 = block_sum(s2, red);
  __syncthreads();
  s3 = block_sum(s3, red);
  const float a = coef[0] / sqrtf(s1 / (float)F + eps), b = coef[1] / sqrtf(s2 / (float)F + eps),
              c3 = coef[2] / sqrtf(s3 / (float)F + eps), e = coef[3];
  for (int c = threadIdx.x; c < F; c += blockDim.x) {
    const float z = to_f32<T>(x[base + c]) + (bias ? to_f32<T>(bias[c]) : 0.f);
    out[base + c] = from_f32<T>(((c3 * z + b) * z + a) * z + e);
  }
}

// The same with the row held in registers between the two passes: VEC channels per 16-byte access, up to CH accesses per
// thread (F <= NT * VEC * CH, NT threads per CTA), the three sums reduced together.
template <typename T, int VEC, int CH, int NT>
__global__ void __launch_bounds__(NT)
power_norm_act_vec_kernel(const T* __restrict__ x, const T* __restrict__ bias, const float* __restrict__ coef,
                          T* __restrict__ out, int F, float eps) {
  __shared__ float red[3][NT / 32];
  struct alignas(16) Pack { T v[VEC]; };
  const long long base = (long long)blockIdx.x * F;
  const int nvec = F / VEC;
  Pack z[CH];
  float s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
  for (int k = 0; k < CH; ++k) {
    const int i = threadIdx.x + k * NT;
    if (i < nvec) {
      z[k] = *reinterpret_cast<const Pack*>(x + base + (long long)i * VEC);
      if (bias != nullptr) {
        const Pack b = *reinterpret_cast<const Pack*>(bias + (long long)i * VEC);
#pragma unroll
        for (int j = 0; j < VEC; ++j) z[k].v[j] = from_f32<T>(to_f32<T>(z[k].v[j]) + to_f32<T>(b.v[j]));
      }
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const float v = to_f32<T>(z[k].v[j]), v2 = v * v;
        s1 += v2, s2 += v2 * v2, s3 += v2 * v2 * v2;
      }
    }
  }
  s1 = warp_sum(s1), s2 = warp_sum(s2), s3 = warp_sum(s3);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[0][w] = s1, red[1][w] = s2, red[2][w] = s3;
  __syncthreads();
  s1 = s2 = s3 = 0.f;
#pragma unroll
  for (int i = 0; i < NT / 32; ++i) s1 += red[0][i], s2 += red[1][i], s3 += red[2][i];
  const float a = coef[0] / sqrtf(s1 / (float)F + eps), b = coef[1] / sqrtf(s2 / (float)F + eps),
              c3 = coef[2] / sqrtf(s3 / (float)F + eps), e = coef[3];
#pragma unroll
  for (int k = 0; k < CH; ++k) {
    const int i = threadIdx.x + k * NT;
    if (i < nvec) {
      Pack o;
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const float v = to_f32<T>(z[k].v[j]);
        o.v[j] = from_f32<T>(((c3 * v + b) * v + a) * v + e);
      }
      *reinterpret_cast<Pack*>(out + base + (long long)i * VEC) = o;
    }
  }
}

// channel_decay_gates with four consecutive key channels (one head: n is a multiple of 4) per thread.
template <typename T>
__global__ void __launch_bounds__(256)
channel_decay_gates_vec_kernel(const T* __restrict__ a_raw, long long lda, const T* __restrict__ b_raw, long long ldb,
                               const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                               float* __restrict__ decay, float* __restrict__ beta, int H, int n, long long total4) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total4) return;
  const int Hn4 = H * n / 4;
  const long long t = i / Hn4;
  const int c = (int)(i % Hn4) * 4, h = c / n;
  struct alignas(sizeof(T) * 4) Pack { T v[4]; };
  const Pack a = *reinterpret_cast<const Pack*>(a_raw + t * lda + c);
  const float4 db = *reinterpret_cast<const float4*>(dt_bias + c);
  const float rate = -expf(A_log[h]);
  float4 o;
  o.x = expf(rate * softplus_f(to_f32<T>(a.v[0]) + db.x));
  o.y = expf(rate * softplus_f(to_f32<T>(a.v[1]) + db.y));
  o.z = expf(rate * softplus_f(to_f32<T>(a.v[2]) + db.z));
  o.w = expf(rate * softplus_f(to_f32<T>(a.v[3]) + db.w));
  *reinterpret_cast<float4*>(decay + t * (long long)H * n + c) = o;
  if (c < H) {
    const int hi = min(c + 4, H);
    for (int j = c; j < hi; ++j) beta[t * H + j] = sigmoid_f(to_f32<T>(b_raw[t * ldb + j]));
  }
}

}  // namespace seqmix
}  // namespace sxb

/* decay fp32 [n_tokens, H * n] = exp(-exp(A_log[h]) * softplus(a_raw + dt_bias)) per head and key channel, beta fp32
 * [n_tokens, H] = sigmoid(b_raw); a_raw `dtype` rows of pitch lda (H * n channels), b_raw `dtype` rows of pitch ldb (H),
 * A_log fp32 [H], dt_bias fp32 [H * n]. */
SXB_API int sxb_channel_decay_gates(const void* a_raw, long long lda, const void* b_raw, long long ldb, const void* A_log,
                                    const void* dt_bias, void* decay, void* beta, int n_tokens, int H, int n, int dtype,
                                    void* stream) {
  const long long total = (long long)n_tokens * H * n;
  if (total <= 0) return SXB_OK;
  const int esz = dtype == 0 ? 4 : 2;
  if (n % 4 == 0 && lda % 4 == 0 && (reinterpret_cast<uintptr_t>(a_raw) % (4 * esz)) == 0 &&
      ((reinterpret_cast<uintptr_t>(dt_bias) | reinterpret_cast<uintptr_t>(decay)) & 15) == 0) {
    const long long total4 = total / 4;
    SEQMIX_DISPATCH(dtype, (channel_decay_gates_vec_kernel<T><<<(unsigned)((total4 + 255) / 256), 256, 0,
                                                               (cudaStream_t)stream>>>(
                               (const T*)a_raw, lda, (const T*)b_raw, ldb, (const float*)A_log, (const float*)dt_bias,
                               (float*)decay, (float*)beta, H, n, total4)));
    SXB_CHECK_LAUNCH();
    return SXB_OK;
  }
  SEQMIX_DISPATCH(dtype, (channel_decay_gates_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
                             (const T*)a_raw, lda, (const T*)b_raw, ldb, (const float*)A_log, (const float*)dt_bias,
                             (float*)decay, (float*)beta, H, n, total)));
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}

/* In place: x `dtype` [rows, width] *= sigmoid(gate[row, c / group]); gate `dtype` rows of pitch ldg with width / group
 * entries (group 1: a gate per channel; group = head size: a gate per head). */
SXB_API int sxb_sigmoid_gate_rows(void* x, const void* gate, long long ldg, long long rows, int width, int group,
                                  int dtype, void* stream) {
  const long long total = rows * width;
  if (total <= 0) return SXB_OK;
  if (group <= 0 || width % group) return SXB_ERR_BAD_ARG;
  const int per = dtype == 0 ? 4 : 8;
  const bool aligned = (reinterpret_cast<uintptr_t>(x) & 15) == 0 && width % per == 0 &&
                       (group == 1 ? (ldg % per == 0 && (reinterpret_cast<uintptr_t>(gate) & 15) == 0) : group % per == 0);
  if (aligned) {
    const long long nv = total / per;
    if (dtype == 0) {
      sigmoid_gate_rows_vec_kernel<float, 4><<<(unsigned)((nv + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
          (float*)x, (const float*)gate, ldg, nv, width / 4, group);
    } else if (dtype == 2) {
      sigmoid_gate_rows_vec_kernel<__nv_bfloat16, 8><<<(unsigned)((nv + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
          (__nv_bfloat16*)x, (const __nv_bfloat16*)gate, ldg, nv, width / 8, group);
    } else {
      return SXB_ERR_UNSUPPORTED;
    }
    SXB_CHECK_LAUNCH();
    return SXB_OK;
  }
  SEQMIX_DISPATCH(dtype, (sigmoid_gate_rows_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
                             (T*)x, (const T*)gate, ldg, total, width, group)));
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}

/* out `dtype` [rows, F]: z = in + bias; p1 z / rms(z) + p2 z^2 / rms(z^2) + p3 z^3 / rms(z^3) + p0 with (p1, p2, p3, p0) = coef
 * fp32 [4] and rms over the row (eps inside the root); bias `dtype` [F] or null. */
SXB_API int sxb_power_norm_act(const void* in, const void* bias, const void* coef, void* out, long long rows, int F,
                               float eps, int dtype, void* stream) {
  if (rows <= 0 || F <= 0) return SXB_OK;
  const int per = dtype == 0 ? 4 : 8;
  const bool aligned = F % per == 0 && ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out) |
                                         reinterpret_cast<uintptr_t>(bias)) & 15) == 0;
  if (aligned && F <= 256 * per * 8 && (dtype == 0 || dtype == 2)) {
    cudaStream_t s = (cudaStream_t)stream;
    const int chunks = (F / per + 255) / 256;
#define POWER_NORM(CH, NT)                                                                                          \
  do {                                                                                                              \
    if (dtype == 0)                                                                                                 \
      power_norm_act_vec_kernel<float, 4, CH, NT><<<(unsigned)rows, NT, 0, s>>>(                                    \
          (const float*)in, (const float*)bias, (const float*)coef, (float*)out, F, eps);                           \
    else                                                                                                            \
      power_norm_act_vec_kernel<__nv_bfloat16, 8, CH, NT><<<(unsigned)rows, NT, 0, s>>>(                            \
          (const __nv_bfloat16*)in, (const __nv_bfloat16*)bias, (const float*)coef, (__nv_bfloat16*)out, F, eps);   \
  } while (0)
    if (chunks <= 1) POWER_NORM(1, 256);
    else if (chunks <= 2) POWER_NORM(2, 256);
    else if (chunks <= 4) POWER_NORM(4, 256);
    else POWER_NORM(4, 512);          // rows of up to 512 * 4 words: twice the threads instead of twice the registers
#undef POWER_NORM
    SXB_CHECK_LAUNCH();
    return SXB_OK;
  }
  SEQMIX_DISPATCH(dtype, (power_norm_act_kernel<T><<<(unsigned)rows, 256, 0, (cudaStream_t)stream>>>(
                             (const T*)in, (const T*)bias, (const float*)coef, (T*)out, F, eps)));
  SXB_CHECK_LAUNCH();
  return SXB_OK;
}
