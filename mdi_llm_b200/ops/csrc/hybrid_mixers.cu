// Kernels of the hybrid (attention + recurrent) model family: packed variable-length batches, slot-indexed state.
//
// A step is a packed batch of N tokens from `nseq` sequences.  `meta[4*s] = {first token row, token count, slot,
// position of the first token}` describes sequence s, `tok_seq[i]` names the sequence of token row i.  The same
// kernels serve prompts (many tokens per sequence) and decoding (one token per sequence): what differs is only
// the meta table.  Every kernel is templated on the activation type (bf16 or fp32); sums, norms, softmax, decays
// and recurrent state are fp32 in both.  This file is compiled WITHOUT fast-math: its exponentials, divisions and
// square roots are the IEEE ones.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace hyb {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ void load8(const float* p, float* f) {
  float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ void load8(const bf16* p, float* f) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

__device__ __forceinline__ void store8(float* p, const float* f) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}
__device__ __forceinline__ void store8(bf16* p, const float* f) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Sum over the block; every thread gets the result.  `red` holds 33 floats.  Safe to call back to back.
__device__ __forceinline__ float block_sum(float v, float* red) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  if (w == 0) {
    float t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float siluf_(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float gelu_erff_(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }

// ---------------------------------------------------------------------------------------------------------
// rows: embedding gather, casts, norms, element-wise epilogues
// ---------------------------------------------------------------------------------------------------------
// x[t] = scale * table[tokens[t]] (+ pos_table[position of t] when the model has learned positions), in fp32.
template <typename T>
__global__ void embed_rows_kernel(const T* __restrict__ table, const int* __restrict__ tokens, float* __restrict__ x,
                                  int C, const T* __restrict__ pos_table, const int* __restrict__ meta,
                                  const int* __restrict__ tok_seq, float scale) {
  int t = blockIdx.x;
  const T* src = table + (size_t)tokens[t] * C;
  float* dst = x + (size_t)t * C;
  if (pos_table) {
    const int* m = meta + 4 * tok_seq[t];
    const T* pr = pos_table + (size_t)(m[3] + (t - m[0])) * C;
    for (int i = threadIdx.x; i < C; i += blockDim.x) dst[i] = scale * to_f(src[i]) + to_f(pr[i]);
    return;
  }
  for (int i = threadIdx.x; i < C; i += blockDim.x) dst[i] = scale * to_f(src[i]);
}

template <typename Tin, typename Tout>
__global__ void cast_rows_kernel(const Tin* __restrict__ in, long long in_stride, Tout* __restrict__ out,
                                 long long out_stride, int n) {
  const Tin* src = in + (size_t)blockIdx.x * in_stride;
  Tout* dst = out + (size_t)blockIdx.x * out_stride;
  for (int i = threadIdx.x; i < n; i += blockDim.x) dst[i] = from_f<Tout>(to_f(src[i]));
}

// kind 0: (x - mean) / sqrt(var + eps) * w + b      kind 1: x / sqrt(mean(x^2) + eps) * w
// kind 2: x (no normalisation).  accumulate != 0: out (fp32) += scale * result, the residual update of a block;
// else out = result.  The weight applied is w_offset + w (w_offset = 1: a weight stored as its deviation from one).
// copy (optional, dense rows of n, with accumulate): the updated residual rounded to the weight's type, which is what
// the next sublayer of a post-norm block reads.
template <typename Tin, typename Tw, typename Tout>
__global__ void norm_rows_kernel(const Tin* __restrict__ in, long long in_stride, const Tw* __restrict__ w,
                                 const Tw* __restrict__ b, Tout* __restrict__ out, long long out_stride, int n,
                                 float eps, int kind, int accumulate, float scale, float w_offset, Tw* __restrict__ copy) {
  __shared__ float red[33];
  const Tin* src = in + (size_t)blockIdx.x * in_stride;
  Tout* dst = out + (size_t)blockIdx.x * out_stride;
  if (kind == 2) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      float y = to_f(src[i]);
      if (accumulate) dst[i] = from_f<Tout>(to_f(dst[i]) + scale * y);
      else dst[i] = from_f<Tout>(y);
    }
    return;
  }
  float mean = 0.f;
  if (kind == 0) {
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) s += to_f(src[i]);
    mean = block_sum(s, red) / n;
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float d = to_f(src[i]) - mean;
    ss += d * d;
  }
  float inv = 1.f / sqrtf(block_sum(ss, red) / n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float y = (to_f(src[i]) - mean) * inv;
    if (w) y *= w_offset + to_f(w[i]);
    if (b) y += to_f(b[i]);
    if (accumulate) {
      float r = to_f(dst[i]) + scale * y;
      dst[i] = from_f<Tout>(r);
      if (copy) copy[(size_t)blockIdx.x * n + i] = from_f<Tw>(r);
    } else {
      dst[i] = from_f<Tout>(y);
    }
  }
}

// act 0: gelu(erf) in place.  act 1: out[r, c] = a[r, c] * sigmoid(g[r, c]) where a is stored head-major
// ([heads, rows, hv]) and out/g are row-major ([rows, heads * hv]).
template <typename T>
__global__ void gelu_rows_kernel(T* __restrict__ x, long long total, int act) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float v = to_f(x[i]);
  if (act == 0) v = gelu_erff_(v);
  else { v = fmaxf(v, 0.f); v = v * v; }  // squared ReLU
  x[i] = from_f<T>(v);
}
template <typename T>
__global__ void headmajor_gate_kernel(const T* __restrict__ a, const T* __restrict__ g, long long g_stride,
                                      T* __restrict__ out, int rows, int heads, int hv) {
  int r = blockIdx.x;
  int n = heads * hv;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    int h = c / hv, d = c - h * hv;
    float v = to_f(a[((size_t)h * rows + r) * hv + d]);
    out[(size_t)r * n + c] = from_f<T>(v * sigmoidf_(to_f(g[(size_t)r * g_stride + c])));
  }
}
template <typename T>
__global__ void softcap_kernel(const T* __restrict__ in, float* __restrict__ out, long long total, float cap) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) {
    float v = to_f(in[i]);
    out[i] = cap > 0.f ? cap * tanhf(v / cap) : v;
  }
}

// ---------------------------------------------------------------------------------------------------------
// latent attention: cache append (norm + rotary) and attention over the shared latent rows
// ---------------------------------------------------------------------------------------------------------
// One block per token.  The row `ckv` holds [L latent | R rotary key]: the latent is RMS-normed with `w`, the key
// part is rotated for the token's position; both go to cache[slot, pos].  The rotary part of each query head
// (last R of its D + R values) is rotated in place.  Pair (i, i + nrot/2), angle = pos * inv_freq[i].
template <typename T>
__global__ void latent_append_kernel(const T* __restrict__ ckv, long long ckv_stride, T* __restrict__ q,
                                     long long q_stride, const T* __restrict__ w, const float* __restrict__ inv_freq,
                                     T* __restrict__ cache, long long slot_stride, const int* __restrict__ meta,
                                     const int* __restrict__ tok_seq, int H, int D, int R, int L, int nrot, float eps) {
  __shared__ float red[33];
  int tok = blockIdx.x;
  const int* m = meta + 4 * tok_seq[tok];
  int pos = m[3] + tok - m[0];
  const T* src = ckv + (size_t)tok * ckv_stride;
  T* dst = cache + (size_t)m[2] * slot_stride + (size_t)pos * (L + R);
  float ss = 0.f;
  for (int i = threadIdx.x; i < L; i += blockDim.x) {
    float v = to_f(src[i]);
    ss += v * v;
  }
  float inv = 1.f / sqrtf(block_sum(ss, red) / L + eps);
  for (int i = threadIdx.x; i < L; i += blockDim.x) dst[i] = from_f<T>(to_f(src[i]) * inv * to_f(w[i]));
  int half = nrot / 2;
  // work items: (H + 1) vectors (vector H is the shared key part) x (half pairs, then the R - nrot values that pass);
  // one thread owns both members of a pair, so the in-place rotation of q needs no barrier
  int per = half + (R - nrot);
  for (int idx = threadIdx.x; idx < (H + 1) * per; idx += blockDim.x) {
    int vec = idx / per, i = idx - vec * per;
    T* qd = q + (size_t)tok * q_stride + (size_t)vec * (D + R) + D;
    const T* s = vec < H ? qd : src + L;
    T* d = vec < H ? qd : dst + L;
    if (i < half) {
      float sn, cs;
      sincosf((float)pos * inv_freq[i], &sn, &cs);
      float u = to_f(s[i]), v = to_f(s[i + half]);
      d[i] = from_f<T>(u * cs - v * sn);
      d[i + half] = from_f<T>(v * cs + u * sn);
    } else if (vec == H) {
      d[nrot + i - half] = s[nrot + i - half];
    }
  }
}

// Attention of H query heads over ONE shared key row per position, whose first Dv entries are also the value
// (queries arrive already multiplied into the latent space).  Block = one token x 8 heads, one warp per head;
// a tile of 32 cached rows is staged in shared memory once and used by all 8 heads.  Online softmax in fp32.
#define LAT_WARPS 8
#define LAT_TILE 32
#define LAT_MAXV 16  // Dv <= 512
template <typename T>
__global__ void latent_attn_kernel(const T* __restrict__ qlat, const T* __restrict__ q, long long q_stride,
                                   const T* __restrict__ cache, long long slot_stride, const int* __restrict__ meta,
                                   const int* __restrict__ tok_seq, T* __restrict__ out, int N, int H, int D, int R,
                                   int L, float scale, int nsplit, float* __restrict__ part_acc,
                                   float* __restrict__ part_ml) {
  extern __shared__ float smem[];
  int Dk = L + R, ldk = Dk + 1;
  float* sq = smem;                       // [LAT_WARPS][Dk]
  float* kt = smem + LAT_WARPS * Dk;      // [LAT_TILE][ldk]
  int tok = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int* m = meta + 4 * tok_seq[tok];
  int nkeys = m[3] + tok - m[0] + 1;
  int h = blockIdx.y * LAT_WARPS + warp;
  bool active = h < H;
  if (active) {
    for (int d = lane; d < Dk; d += 32) {
      float v = d < L ? to_f(qlat[((size_t)h * N + tok) * L + d])
                      : to_f(q[(size_t)tok * q_stride + (size_t)h * (D + R) + D + (d - L)]);
      sq[warp * Dk + d] = v * scale;
    }
  }
  const T* rows = cache + (size_t)m[2] * slot_stride;
  float mx = -INFINITY, l = 0.f, acc[LAT_MAXV];
#pragma unroll
  for (int i = 0; i < LAT_MAXV; ++i) acc[i] = 0.f;
  int nv = (L + 31) / 32;
  // with nsplit > 1 (few query tokens, long contexts) block z scans only its share of the keys and leaves an
  // unnormalised partial result; latent_combine_kernel merges the shares
  int chunk = ((nkeys + nsplit - 1) / nsplit + LAT_TILE - 1) / LAT_TILE * LAT_TILE;
  int k_begin = blockIdx.z * chunk, k_end = min(nkeys, k_begin + chunk);
  __syncthreads();
  for (int t0 = k_begin; t0 < k_end; t0 += LAT_TILE) {
    __syncthreads();
    int lim = min(LAT_TILE, k_end - t0);
    if ((Dk & 7) == 0 && (((size_t)rows) & 15) == 0) {  // 8 values per load (16 bytes of bf16, 2 x 16 of fp32)
      int per = Dk >> 3;
      for (int idx = threadIdx.x; idx < lim * per; idx += blockDim.x) {
        int jj = idx / per, d = (idx - jj * per) << 3;
        float f[8];
        load8(rows + (size_t)(t0 + jj) * Dk + d, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) kt[jj * ldk + d + e] = f[e];
      }
    } else {
      for (int idx = threadIdx.x; idx < lim * Dk; idx += blockDim.x) {
        int jj = idx / Dk, d = idx - jj * Dk;
        kt[jj * ldk + d] = to_f(rows[(size_t)(t0 + jj) * Dk + d]);
      }
    }
    __syncthreads();
    if (!active) continue;
    float s = -INFINITY;
    if (lane < lim) {
      s = 0.f;
      const float* qv = sq + warp * Dk;
      const float* kv = kt + lane * ldk;
      for (int d = 0; d < Dk; ++d) s += qv[d] * kv[d];
    }
    float mnew = fmaxf(mx, warp_max(s));
    float corr = expf(mx - mnew);
    float p = lane < lim ? expf(s - mnew) : 0.f;
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < LAT_MAXV; ++i) acc[i] *= corr;
    for (int jj = 0; jj < lim; ++jj) {
      float pj = __shfl_sync(0xffffffffu, p, jj);
      const float* kv = kt + jj * ldk;
#pragma unroll
      for (int i = 0; i < LAT_MAXV; ++i)
        if (i < nv) {
          int d = lane + 32 * i;
          if (d < L) acc[i] += pj * kv[d];
        }
    }
    mx = mnew;
  }
  if (active && nsplit == 1) {
#pragma unroll
    for (int i = 0; i < LAT_MAXV; ++i)
      if (i < nv) {
        int d = lane + 32 * i;
        if (d < L) out[((size_t)h * N + tok) * L + d] = from_f<T>(acc[i] / l);
      }
  } else if (active) {
    size_t base = ((size_t)blockIdx.z * H + h) * N + tok;
#pragma unroll
    for (int i = 0; i < LAT_MAXV; ++i)
      if (i < nv) {
        int d = lane + 32 * i;
        if (d < L) part_acc[base * L + d] = acc[i];
      }
    if (lane == 0) {
      part_ml[base * 2] = mx;
      part_ml[base * 2 + 1] = l;
    }
  }
}

// out[h, tok] = sum_z acc_z e^(m_z - m) / sum_z l_z e^(m_z - m), m = max_z m_z (an empty share has m = -inf, l = 0)
template <typename T>
__global__ void latent_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                      T* __restrict__ out, int N, int H, int L, int nsplit) {
  int tok = blockIdx.x, h = blockIdx.y;
  float m = -INFINITY;
  for (int z = 0; z < nsplit; ++z) m = fmaxf(m, part_ml[(((size_t)z * H + h) * N + tok) * 2]);
  float den = 0.f;
  for (int z = 0; z < nsplit; ++z) {
    size_t b = ((size_t)z * H + h) * N + tok;
    float lz = part_ml[b * 2 + 1];
    if (lz > 0.f) den += lz * expf(part_ml[b * 2] - m);
  }
  for (int d = threadIdx.x; d < L; d += blockDim.x) {
    float num = 0.f;
    for (int z = 0; z < nsplit; ++z) {
      size_t b = ((size_t)z * H + h) * N + tok;
      if (part_ml[b * 2 + 1] > 0.f) num += part_acc[b * L + d] * expf(part_ml[b * 2] - m);
    }
    out[((size_t)h * N + tok) * L + d] = from_f<T>(num / den);
  }
}

// Causal softmax of fp32 score rows for the expanded (prompt) form of latent attention: row (h, i) sees keys
// j <= first_pos + i; p = softmax(scale * s) over those, zeros elsewhere, written in the activation type.
// sink != 0: one more slot of score zero joins the denominator (it has no value): p_j = e^{s_j} / (1 + sum e^{s_k}).
// split != 0: a row of p is 2 * keys wide: the weights rounded to T, and behind them the remainders (weight minus its
// rounding) rounded to T, so that a matrix product with the values stacked twice sums the weights to 16 mantissa bits.
// cap > 0: the scaled score becomes cap * tanh(scaled score / cap) before the softmax (the transform is applied where a
// score is read; from there on the scale is 1).  sink_vals (with sink != 0): the sink's score is sink_vals[head]
// instead of zero, head = (row / rows_per_head) % sink_heads; it is neither scaled nor capped.
#define CS_CACHE 8  // scores a thread keeps in registers: rows of up to 8 * 256 keys are read once
template <typename T>
__global__ void causal_softmax_kernel(const float* __restrict__ s, T* __restrict__ p, int rows_per_head, int keys,
                                      int first_pos, float scale, int window, int key0, int sink, int split,
                                      float cap, const float* __restrict__ sink_vals, int sink_heads) {
  __shared__ float red[33];
  size_t row = blockIdx.x;
  int i = (int)(row % rows_per_head);
  const float raw_scale = scale, inv_cap = cap > 0.f ? 1.f / cap : 0.f;
  if (cap > 0.f) scale = 1.f;
#define CS_SCORE(x) (cap > 0.f ? cap * tanhf((x) * raw_scale * inv_cap) : (x))
  // the sink's score in the units of the stored scores (they are multiplied by `scale` inside the exponent)
  const float sink_raw = sink && sink_vals ? sink_vals[(row / rows_per_head) % sink_heads] / scale : 0.f;
  int pos = first_pos + i;  // column j is position key0 + j; visible: pos - window < key0 + j <= pos
  int vis = max(0, min(keys, pos - key0 + 1));
  int lo = window > 0 ? max(0, pos - window + 1 - key0) : 0;
  const float* src = s + row * keys;
  T* dst = p + row * (split ? 2 * (size_t)keys : (size_t)keys);
  bool cached = keys <= CS_CACHE * (int)blockDim.x;  // the same for every thread of the block
  float v[CS_CACHE];
  float m = -INFINITY;
  if (cached && (keys & 7) == 0) {
    // rows of a multiple of 8 keys: a thread owns 8 neighbouring keys, read with two 16-byte loads and written with
    // one (bf16) or two (fp32) 16-byte stores per output; threads past the row's end only take part in the sums
    int j0 = threadIdx.x * 8;
    bool mine = j0 < keys;
    if (mine) load8(src + j0, v);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      int j = j0 + c;
      v[c] = mine && j >= lo && j < vis ? CS_SCORE(v[c]) : -INFINITY;
      m = fmaxf(m, v[c]);
    }
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    m = -INFINITY;
    for (int w = 0; w < (blockDim.x + 31) / 32; ++w) m = fmaxf(m, red[w]);
    if (sink) m = fmaxf(m, sink_raw);
    float sum = 0.f;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      v[c] = v[c] == -INFINITY ? 0.f : expf((v[c] - m) * scale);
      sum += v[c];
    }
    sum = block_sum(sum, red);
    if (sink) sum += expf((sink_raw - m) * scale);
    float inv = 1.f / sum;
    if (!mine) return;
    float rest[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      v[c] = v[c] == 0.f ? 0.f : v[c] * inv;
      rest[c] = v[c] - to_f(from_f<T>(v[c]));
    }
    store8(dst + j0, v);
    if (split) store8(dst + keys + j0, rest);
    return;
  }
  if (cached) {
#pragma unroll
    for (int c = 0; c < CS_CACHE; ++c) {
      int j = threadIdx.x + c * blockDim.x;
      v[c] = j >= lo && j < vis ? CS_SCORE(src[j]) : -INFINITY;
      m = fmaxf(m, v[c]);
    }
  } else {
    for (int j = lo + threadIdx.x; j < vis; j += blockDim.x) m = fmaxf(m, CS_SCORE(src[j]));
  }
  m = warp_max(m);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  m = -INFINITY;
  for (int w = 0; w < (blockDim.x + 31) / 32; ++w) m = fmaxf(m, red[w]);
  if (sink) m = fmaxf(m, sink_raw);  // scale > 0: the shift that keeps every exponent <= 0
  float sum = 0.f;
  if (cached) {
#pragma unroll
    for (int c = 0; c < CS_CACHE; ++c) {
      v[c] = v[c] == -INFINITY ? 0.f : expf((v[c] - m) * scale);  // hidden keys: weight zero
      sum += v[c];
    }
  } else {
    for (int j = lo + threadIdx.x; j < vis; j += blockDim.x) sum += expf((CS_SCORE(src[j]) - m) * scale);
  }
  sum = block_sum(sum, red);
  if (sink) sum += expf((sink_raw - m) * scale);
  float inv = 1.f / sum;
  if (cached) {
#pragma unroll
    for (int c = 0; c < CS_CACHE; ++c) {
      int j = threadIdx.x + c * blockDim.x;
      if (j < keys) {
        float w = v[c] == 0.f ? 0.f : v[c] * inv;  // a row without a visible key and without a sink: inv is infinite
        T hi = from_f<T>(w);
        dst[j] = hi;
        if (split) dst[keys + j] = from_f<T>(w - to_f(hi));
      }
    }
    return;
  }
  for (int j = threadIdx.x; j < keys; j += blockDim.x) {
    float w = j >= lo && j < vis ? expf((CS_SCORE(src[j]) - m) * scale) * inv : 0.f;
    T hi = from_f<T>(w);
    dst[j] = hi;
    if (split) dst[keys + j] = from_f<T>(w - to_f(hi));
  }
#undef CS_SCORE
}

// ---------------------------------------------------------------------------------------------------------
// short causal convolution + SiLU over packed sequences, with the last taps-1 inputs kept per slot
// ---------------------------------------------------------------------------------------------------------
// y[t, c] = silu(sum_j w[c, j] * x[t - (taps-1-j), c]); inputs before this step come from state[slot]
// ([taps-1, C], oldest first; zero for a fresh slot).
template <typename T>
__global__ void conv_silu_kernel(const T* __restrict__ x, long long x_stride, const T* __restrict__ w,
                                 const T* __restrict__ state, T* __restrict__ y, long long y_stride,
                                 const int* __restrict__ meta, const int* __restrict__ tok_seq, int C, int taps) {
  int tok = blockIdx.x;
  const int* m = meta + 4 * tok_seq[tok];
  int local = tok - m[0];
  const T* st = state + (size_t)m[2] * (taps - 1) * C;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
      int src = local - (taps - 1 - j);
      float v = src >= 0 ? to_f(x[(size_t)(m[0] + src) * x_stride + c]) : to_f(st[(size_t)(taps - 1 + src) * C + c]);
      acc += to_f(w[(size_t)c * taps + j]) * v;
    }
    y[(size_t)tok * y_stride + c] = from_f<T>(siluf_(acc));
  }
}
// After the convolution: state[slot] <- the last taps-1 inputs of the sequence (old rows shift up when the step
// brought fewer than taps-1 tokens).  One thread per channel walks the rows oldest first, so it never reads a row
// it has already overwritten.
template <typename T>
__global__ void conv_state_kernel(const T* __restrict__ x, long long x_stride, T* __restrict__ state,
                                  const int* __restrict__ meta, int C, int taps) {
  const int* m = meta + 4 * blockIdx.x;
  int n = m[1], keep = taps - 1;
  T* st = state + (size_t)m[2] * keep * C;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    for (int j = 0; j < keep; ++j) {
      int src = n - keep + j;  // local index of the input that becomes row j
      st[(size_t)j * C + c] = src >= 0 ? x[(size_t)(m[0] + src) * x_stride + c] : st[(size_t)(j + n) * C + c];
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// gated linear recurrences with a [D, V] state per head (fp32, in shared memory while a step runs)
// ---------------------------------------------------------------------------------------------------------
// mode 0 (gated linear attention): a = exp(-softplus(-(z + zb)) / tau);  S = a S + k v^T;  o = S^T (q D^-1/2)
// mode 1 (gated delta rule):       a = exp(-exp(A_log[h]) softplus(z + zb)); q, k unit vectors (eps 1e-6);
//                                  S = a S; u = beta (v - S^T k); S += k u^T; o = S^T (q D^-1/2)
// then o / rms(o) * w * gate, gate = silu(g) (mode 0) or sigmoid(g) (mode 1).
// Block = one (sequence, head), one thread per value column: columns never interact inside the recurrence.
struct RecArgs {
  const void *q, *k, *v, *z, *g, *beta, *zb, *a_log, *w;
  void* out;
  float* state;
  const int* meta;
  long long q_stride, k_stride, v_stride, z_stride, g_stride, beta_stride, out_stride;
  int H, G, D, V, mode;
  float tau, eps;
};

template <typename T>
__global__ void gated_recurrence_kernel(RecArgs a) {
  extern __shared__ float smem[];
  int D = a.D, V = a.V, h = blockIdx.y, j = threadIdx.x;
  float* S = smem;            // [D][V]
  float* sq = S + D * V;      // [D]
  float* sk = sq + D;
  float* sa = sk + D;
  float* red = sa + D;        // [33]
  const int* m = a.meta + 4 * blockIdx.x;
  int start = m[0], n = m[1];
  float* gS = a.state + ((size_t)m[2] * a.H + h) * D * V;
  for (int i = threadIdx.x; i < D * V; i += blockDim.x) S[i] = gS[i];
  int kvh = h / (a.H / a.G);
  const T *q = (const T*)a.q, *k = (const T*)a.k, *v = (const T*)a.v, *z = (const T*)a.z, *g = (const T*)a.g;
  const T *beta = (const T*)a.beta, *zb = (const T*)a.zb, *w = (const T*)a.w, *alog = (const T*)a.a_log;
  T* out = (T*)a.out;
  float rate = a.mode == 1 ? expf(to_f(alog[h])) : 0.f;
  float dscale = 1.f / sqrtf((float)D);
  for (int t = 0; t < n; ++t) {
    size_t row = (size_t)start + t;
    float pq = 0.f, pk = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
      float qv = to_f(q[row * a.q_stride + kvh * D + i]);
      float kv = to_f(k[row * a.k_stride + kvh * D + i]);
      float zz = to_f(z[row * a.z_stride + h * D + i]) + (zb ? to_f(zb[h * D + i]) : 0.f);
      sq[i] = qv;
      sk[i] = kv;
      sa[i] = a.mode == 1 ? expf(-rate * softplusf_(zz)) : expf(-softplusf_(-zz) / a.tau);
      pq += qv * qv;
      pk += kv * kv;
    }
    float qs = dscale, ks = 1.f;
    if (a.mode == 1) {
      float sumq = block_sum(pq, red);
      float sumk = block_sum(pk, red);
      qs = dscale / sqrtf(sumq + 1e-6f);
      ks = 1.f / sqrtf(sumk + 1e-6f);
    } else {
      __syncthreads();
    }
    float o = 0.f;
    if (j < V) {
      float u = to_f(v[row * a.v_stride + h * V + j]);
      if (a.mode == 1) {
        float r = 0.f;
        for (int i = 0; i < D; ++i) r += sa[i] * S[i * V + j] * (sk[i] * ks);
        u = sigmoidf_(to_f(beta[row * a.beta_stride + h])) * (u - r);
      }
      for (int i = 0; i < D; ++i) {
        float s = sa[i] * S[i * V + j] + (sk[i] * ks) * u;
        S[i * V + j] = s;
        o += s * (sq[i] * qs);
      }
    }
    float ss = block_sum(j < V ? o * o : 0.f, red);
    if (j < V) {
      float y = o / sqrtf(ss / V + a.eps) * to_f(w[j]);
      float gv = to_f(g[row * a.g_stride + h * V + j]);
      y *= a.mode == 1 ? sigmoidf_(gv) : siluf_(gv);
      out[row * a.out_stride + h * V + j] = from_f<T>(y);
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < D * V; i += blockDim.x) gS[i] = S[i];
}

// The same recurrence with the state in registers: R lanes of a warp share one value column and own every R-th
// key row of it (<= ROWS rows each), partial sums meet through shuffles.  The sequential chain per token is D/R
// instead of D steps and the state never touches shared memory.  Per token one thread per key channel prepares
// {decay, k, q, decay*k} (unit-normed and scaled) as ONE 16-byte shared-memory word, so each step of the two row
// loops is a single LDS.128.  The next token's inputs are requested before the current one is computed and stay in
// their storage type until used (a conversion right after the load would stall the in-order warp on it).
// Lanes are laid out [row group][column] inside a warp: a state row is touched 32/R columns at a time.
template <typename T, int R, int ROWS>
__global__ void __launch_bounds__(ROWS > 16 ? 512 : 1024) gated_recurrence_reg_kernel(RecArgs a) {
  constexpr int CPW = 32 / R;
  extern __shared__ float4 smem4[];
  int D = a.D, V = a.V, h = blockIdx.y;
  float4* sp = smem4;                 // [D] {decay, k, q, decay * k}
  float* red = (float*)(smem4 + D);   // [33]
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int r = lane / CPW, j = warp * CPW + (lane % CPW);
  bool col = j < V;
  const int* m = a.meta + 4 * blockIdx.x;
  int start = m[0], n = m[1];
  float* gS = a.state + ((size_t)m[2] * a.H + h) * D * V;
  float s[ROWS];
#pragma unroll
  for (int ii = 0; ii < ROWS; ++ii) {
    int i = r + R * ii;
    s[ii] = (col && i < D) ? gS[(size_t)i * V + j] : 0.f;
  }
  int kvh = h / (a.H / a.G);
  const T *q = (const T*)a.q, *k = (const T*)a.k, *v = (const T*)a.v, *z = (const T*)a.z, *g = (const T*)a.g;
  const T *beta = (const T*)a.beta, *zb = (const T*)a.zb, *w = (const T*)a.w, *alog = (const T*)a.a_log;
  T* out = (T*)a.out;
  float rate = a.mode == 1 ? expf(to_f(alog[h])) : 0.f;
  float dscale = 1.f / sqrtf((float)D);
  int i0 = threadIdx.x;
  bool has0 = i0 < D, lead = col && r == 0;  // the launcher guarantees D <= blockDim.x
  T nq = from_f<T>(0.f), nk = nq, nz = nq, nu = nq, ng = nq, nb = nq;
  float zb0 = (has0 && zb) ? to_f(zb[h * D + i0]) : 0.f;
  float wj = lead ? to_f(w[j]) : 0.f;
  auto fetch = [&](int t) {
    size_t row = (size_t)start + t;
    if (has0) {
      nq = q[row * a.q_stride + kvh * D + i0];
      nk = k[row * a.k_stride + kvh * D + i0];
      nz = z[row * a.z_stride + h * D + i0];
    }
    if (col) nu = v[row * a.v_stride + h * V + j];
    if (lead) ng = g[row * a.g_stride + h * V + j];
    if (a.mode == 1) nb = beta[row * a.beta_stride + h];
  };
  if (n > 0) fetch(0);
  for (int t = 0; t < n; ++t) {
    size_t row = (size_t)start + t;
    float cq = to_f(nq), ck = to_f(nk), cz = to_f(nz), u = col ? to_f(nu) : 0.f, gv = to_f(ng), bt = to_f(nb);
    if (t + 1 < n) fetch(t + 1);
    float dec = 0.f;
    if (has0) {
      float zz = cz + zb0;
      dec = a.mode == 1 ? expf(-rate * softplusf_(zz)) : expf(-softplusf_(-zz) / a.tau);
    }
    float qs = dscale, ks = 1.f;
    if (a.mode == 1) {
      float sumq = block_sum(has0 ? cq * cq : 0.f, red);
      float sumk = block_sum(has0 ? ck * ck : 0.f, red);
      qs = dscale / sqrtf(sumq + 1e-6f);
      ks = 1.f / sqrtf(sumk + 1e-6f);
    }
    if (has0) sp[i0] = make_float4(dec, ck * ks, cq * qs, dec * (ck * ks));
    __syncthreads();
    if (a.mode == 1) {
      float rp = 0.f;
#pragma unroll
      for (int ii = 0; ii < ROWS; ++ii) {
        int i = r + R * ii;
        if (i < D) rp += s[ii] * sp[i].w;
      }
#pragma unroll
      for (int o = CPW; o < 32; o <<= 1) rp += __shfl_xor_sync(0xffffffffu, rp, o);
      u = sigmoidf_(bt) * (u - rp);
    }
    float o = 0.f;
#pragma unroll
    for (int ii = 0; ii < ROWS; ++ii) {
      int i = r + R * ii;
      if (i < D) {
        float4 c = sp[i];
        float sv = c.x * s[ii] + c.y * u;
        s[ii] = sv;
        o += sv * c.z;
      }
    }
#pragma unroll
    for (int off = CPW; off < 32; off <<= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
    float ss = block_sum(lead ? o * o : 0.f, red);  // its barriers also fence sp before the next token rewrites it
    if (lead) {
      float y = o / sqrtf(ss / V + a.eps) * wj;
      y *= a.mode == 1 ? sigmoidf_(gv) : siluf_(gv);
      out[row * a.out_stride + h * V + j] = from_f<T>(y);
    }
  }
#pragma unroll
  for (int ii = 0; ii < ROWS; ++ii) {
    int i = r + R * ii;
    if (col && i < D) gS[(size_t)i * V + j] = s[ii];
  }
}

// ---- prompts: the recurrence as three kernels, so that the sequential part holds nothing but the recurrence ----
// (1) rec_prep: everything that does not depend on the state, for all tokens in parallel: decay, unit-normed and
//     scaled q and k, decay * k as one float4 per (token, head, key channel); sigmoid(beta) per (token, head).
// (2) rec_scan: the scan itself.  Value columns never interact, so a head's columns are spread over blockIdx.z
//     blocks (more SMs busy, fewer warps per step); per token: stage D float4 (double-buffered, ONE barrier),
//     two short row loops from registers, shuffles, raw fp32 read-out.
// (3) rec_finish: per (token, head) RMS norm of the read-out, weight, gate, cast — parallel over tokens again.
template <typename T>
__global__ void rec_prep_kernel(RecArgs a, float4* __restrict__ prep, float* __restrict__ bsig) {
  __shared__ float red[33];
  int tok = blockIdx.x, h = blockIdx.y, D = a.D;
  int kvh = h / (a.H / a.G);
  const T *q = (const T*)a.q, *k = (const T*)a.k, *z = (const T*)a.z, *zb = (const T*)a.zb;
  float rate = a.mode == 1 ? expf(to_f(((const T*)a.a_log)[h])) : 0.f;
  float pq = 0.f, pk = 0.f;
  if (a.mode == 1) {
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
      float qv = to_f(q[(size_t)tok * a.q_stride + kvh * D + i]), kv = to_f(k[(size_t)tok * a.k_stride + kvh * D + i]);
      pq += qv * qv;
      pk += kv * kv;
    }
    pq = block_sum(pq, red);
    pk = block_sum(pk, red);
  }
  float dscale = 1.f / sqrtf((float)D);
  float qs = a.mode == 1 ? dscale / sqrtf(pq + 1e-6f) : dscale;
  float ks = a.mode == 1 ? 1.f / sqrtf(pk + 1e-6f) : 1.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float qv = to_f(q[(size_t)tok * a.q_stride + kvh * D + i]), kv = to_f(k[(size_t)tok * a.k_stride + kvh * D + i]);
    float zz = to_f(z[(size_t)tok * a.z_stride + h * D + i]) + (zb ? to_f(zb[h * D + i]) : 0.f);
    float dec = a.mode == 1 ? expf(-rate * softplusf_(zz)) : expf(-softplusf_(-zz) / a.tau);
    prep[((size_t)tok * a.H + h) * D + i] = make_float4(dec, kv * ks, qv * qs, dec * (kv * ks));
  }
  if (a.mode == 1 && threadIdx.x == 0)
    bsig[(size_t)tok * a.H + h] = sigmoidf_(to_f(((const T*)a.beta)[(size_t)tok * a.beta_stride + h]));
}

template <typename T, int R>
__global__ void __launch_bounds__(256) rec_scan_kernel(RecArgs a, const float4* __restrict__ prep,
                                                       const float* __restrict__ bsig, float* __restrict__ oraw,
                                                       int cols_per_block) {
  constexpr int CPW = 32 / R;
  constexpr int ROWS = 16;
  extern __shared__ float4 smem4[];  // [2][D]
  int D = a.D, V = a.V, h = blockIdx.y;
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int r = lane / CPW, jl = warp * CPW + (lane % CPW);
  int j = blockIdx.z * cols_per_block + jl;
  bool col = jl < cols_per_block && j < V;
  bool lead = col && r == 0;
  const int* m = a.meta + 4 * blockIdx.x;
  int start = m[0], n = m[1];
  float* gS = a.state + ((size_t)m[2] * a.H + h) * D * V;
  float s[ROWS];
#pragma unroll
  for (int ii = 0; ii < ROWS; ++ii) {
    int i = r + R * ii;
    s[ii] = (col && i < D) ? gS[(size_t)i * V + j] : 0.f;
  }
  const T* v = (const T*)a.v;
  int i0 = threadIdx.x;
  bool has0 = i0 < D;  // the launcher guarantees D <= blockDim.x
  float4 n4 = make_float4(0.f, 0.f, 0.f, 0.f);
  T nu = from_f<T>(0.f);
  float nb = 0.f;
  auto fetch = [&](int t) {
    size_t row = (size_t)start + t;
    if (has0) n4 = prep[(row * a.H + h) * D + i0];
    if (col) nu = v[row * a.v_stride + h * V + j];
    if (a.mode == 1) nb = bsig[row * a.H + h];
  };
  if (n > 0) fetch(0);
  for (int t = 0; t < n; ++t) {
    size_t row = (size_t)start + t;
    float4* sp = smem4 + (t & 1) * D;
    if (has0) sp[i0] = n4;
    float u = col ? to_f(nu) : 0.f, bt = nb;
    if (t + 1 < n) fetch(t + 1);
    __syncthreads();  // the only barrier per token: the other buffer was last read before the previous barrier
    if (a.mode == 1) {
      float rp = 0.f;
#pragma unroll
      for (int ii = 0; ii < ROWS; ++ii) {
        int i = r + R * ii;
        if (i < D) rp += s[ii] * sp[i].w;
      }
#pragma unroll
      for (int o = CPW; o < 32; o <<= 1) rp += __shfl_xor_sync(0xffffffffu, rp, o);
      u = bt * (u - rp);
    }
    float o = 0.f;
#pragma unroll
    for (int ii = 0; ii < ROWS; ++ii) {
      int i = r + R * ii;
      if (i < D) {
        float4 c = sp[i];
        float sv = c.x * s[ii] + c.y * u;
        s[ii] = sv;
        o += sv * c.z;
      }
    }
#pragma unroll
    for (int off = CPW; off < 32; off <<= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
    if (lead) oraw[row * ((size_t)a.H * V) + h * V + j] = o;
  }
#pragma unroll
  for (int ii = 0; ii < ROWS; ++ii) {
    int i = r + R * ii;
    if (col && i < D) gS[(size_t)i * V + j] = s[ii];
  }
}

template <typename T>
__global__ void rec_finish_kernel(RecArgs a, const float* __restrict__ oraw) {
  __shared__ float red[33];
  int tok = blockIdx.x, h = blockIdx.y, V = a.V;
  const float* o = oraw + (size_t)tok * a.H * V + h * V;
  const T *g = (const T*)a.g, *w = (const T*)a.w;
  T* out = (T*)a.out;
  float ss = 0.f;
  for (int j = threadIdx.x; j < V; j += blockDim.x) ss += o[j] * o[j];
  ss = block_sum(ss, red);
  float inv = 1.f / sqrtf(ss / V + a.eps);
  for (int j = threadIdx.x; j < V; j += blockDim.x) {
    float gv = to_f(g[(size_t)tok * a.g_stride + h * V + j]);
    float y = o[j] * inv * to_f(w[j]) * (a.mode == 1 ? sigmoidf_(gv) : siluf_(gv));
    out[(size_t)tok * a.out_stride + h * V + j] = from_f<T>(y);
  }
}

}  // namespace hyb

using namespace hyb;

#define HYB_DISPATCH(dt, expr_bf16, expr_f32) \
  do {                                        \
    if ((dt) == 0) { expr_bf16; } else { expr_f32; } \
  } while (0)

extern "C" {

// dtype codes: 0 = bf16, 1 = fp32
int hyb_embed_rows(const void* table, const int* tokens, float* x, int N, int C, const void* pos_table,
                   const int* meta, const int* tok_seq, float scale, int dt, cudaStream_t st) {
  if (N == 0) return 0;
  if (pos_table && (!meta || !tok_seq)) return -2;
  HYB_DISPATCH(dt,
               (embed_rows_kernel<bf16><<<N, 256, 0, st>>>((const bf16*)table, tokens, x, C, (const bf16*)pos_table, meta,
                                                           tok_seq, scale)),
               (embed_rows_kernel<float><<<N, 256, 0, st>>>((const float*)table, tokens, x, C, (const float*)pos_table,
                                                            meta, tok_seq, scale)));
  return (int)cudaGetLastError();
}

int hyb_cast_rows(const void* in, long long in_stride, int in_dt, void* out, long long out_stride, int out_dt, int rows,
                  int n, cudaStream_t st) {
  if (rows == 0) return 0;
  if (in_dt == 1 && out_dt == 0)
    cast_rows_kernel<float, bf16><<<rows, 256, 0, st>>>((const float*)in, in_stride, (bf16*)out, out_stride, n);
  else if (in_dt == 1 && out_dt == 1)
    cast_rows_kernel<float, float><<<rows, 256, 0, st>>>((const float*)in, in_stride, (float*)out, out_stride, n);
  else if (in_dt == 0 && out_dt == 1)
    cast_rows_kernel<bf16, float><<<rows, 256, 0, st>>>((const bf16*)in, in_stride, (float*)out, out_stride, n);
  else
    cast_rows_kernel<bf16, bf16><<<rows, 256, 0, st>>>((const bf16*)in, in_stride, (bf16*)out, out_stride, n);
  return (int)cudaGetLastError();
}

// w/b have dtype w_dt; in has in_dt; out has out_dt.  Supported (in, w, out): all fp32, or w bf16 with in/out in
// {bf16, fp32}.
int hyb_norm_rows(const void* in, long long in_stride, int in_dt, const void* w, const void* b, int w_dt, void* out,
                  long long out_stride, int out_dt, int rows, int n, float eps, int kind, int accumulate, float scale,
                  float w_offset, void* copy, cudaStream_t st) {
  if (rows == 0) return 0;
  if (copy && (!accumulate || kind == 2)) return -2;
#define NR(TI, TW, TO)                                                                                              \
  norm_rows_kernel<TI, TW, TO><<<rows, 256, 0, st>>>((const TI*)in, in_stride, (const TW*)w, (const TW*)b, (TO*)out, \
                                                      out_stride, n, eps, kind, accumulate, scale, w_offset, (TW*)copy)
  if (w_dt == 1) {
    if (in_dt != 1 || out_dt != 1) return -3;
    NR(float, float, float);
  } else if (in_dt == 1 && out_dt == 0) NR(float, bf16, bf16);
  else if (in_dt == 0 && out_dt == 1) NR(bf16, bf16, float);
  else if (in_dt == 0 && out_dt == 0) NR(bf16, bf16, bf16);
  else NR(float, bf16, float);
#undef NR
  return (int)cudaGetLastError();
}

int hyb_gelu_rows(void* x, long long total, int dt, int act, cudaStream_t st) {
  if (total == 0) return 0;
  int blocks = (int)((total + 255) / 256);
  HYB_DISPATCH(dt, (gelu_rows_kernel<bf16><<<blocks, 256, 0, st>>>((bf16*)x, total, act)),
               (gelu_rows_kernel<float><<<blocks, 256, 0, st>>>((float*)x, total, act)));
  return (int)cudaGetLastError();
}

int hyb_headmajor_gate(const void* a, const void* g, long long g_stride, void* out, int rows, int heads, int hv, int dt,
                       cudaStream_t st) {
  if (rows == 0) return 0;
  HYB_DISPATCH(dt,
               (headmajor_gate_kernel<bf16><<<rows, 256, 0, st>>>((const bf16*)a, (const bf16*)g, g_stride, (bf16*)out,
                                                                  rows, heads, hv)),
               (headmajor_gate_kernel<float><<<rows, 256, 0, st>>>((const float*)a, (const float*)g, g_stride,
                                                                   (float*)out, rows, heads, hv)));
  return (int)cudaGetLastError();
}

int hyb_softcap(const void* in, float* out, long long total, float cap, int dt, cudaStream_t st) {
  if (total == 0) return 0;
  int blocks = (int)((total + 255) / 256);
  HYB_DISPATCH(dt, (softcap_kernel<bf16><<<blocks, 256, 0, st>>>((const bf16*)in, out, total, cap)),
               (softcap_kernel<float><<<blocks, 256, 0, st>>>((const float*)in, out, total, cap)));
  return (int)cudaGetLastError();
}

int hyb_latent_append(const void* ckv, long long ckv_stride, void* q, long long q_stride, const void* w,
                      const float* inv_freq, void* cache, long long slot_stride, const int* meta, const int* tok_seq,
                      int N, int H, int D, int R, int L, int nrot, float eps, int dt, cudaStream_t st) {
  if (N == 0) return 0;
  if (nrot > R || (nrot & 1)) return -2;
  int threads = 256;
  HYB_DISPATCH(dt,
               (latent_append_kernel<bf16><<<N, threads, 0, st>>>((const bf16*)ckv, ckv_stride, (bf16*)q, q_stride,
                                                                  (const bf16*)w, inv_freq, (bf16*)cache, slot_stride,
                                                                  meta, tok_seq, H, D, R, L, nrot, eps)),
               (latent_append_kernel<float><<<N, threads, 0, st>>>((const float*)ckv, ckv_stride, (float*)q, q_stride,
                                                                   (const float*)w, inv_freq, (float*)cache,
                                                                   slot_stride, meta, tok_seq, H, D, R, L, nrot, eps)));
  return (int)cudaGetLastError();
}

int hyb_latent_attn(const void* qlat, const void* q, long long q_stride, const void* cache, long long slot_stride,
                    const int* meta, const int* tok_seq, void* out, int N, int H, int D, int R, int L, float scale,
                    int nsplit, float* part_acc, float* part_ml, int dt, cudaStream_t st) {
  if (N == 0) return 0;
  if (L > 32 * LAT_MAXV || nsplit < 1 || (nsplit > 1 && (!part_acc || !part_ml))) return -3;
  int Dk = L + R;
  size_t smem = (size_t)(LAT_WARPS * Dk + LAT_TILE * (Dk + 1)) * sizeof(float);
  if (smem > 200 * 1024) return -3;
  dim3 grid(N, (H + LAT_WARPS - 1) / LAT_WARPS, nsplit);
  if (dt == 0) {
    cudaFuncSetAttribute(latent_attn_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    latent_attn_kernel<bf16><<<grid, LAT_WARPS * 32, smem, st>>>((const bf16*)qlat, (const bf16*)q, q_stride,
                                                                 (const bf16*)cache, slot_stride, meta, tok_seq,
                                                                 (bf16*)out, N, H, D, R, L, scale, nsplit, part_acc,
                                                                 part_ml);
    if (nsplit > 1) latent_combine_kernel<bf16><<<dim3(N, H), 128, 0, st>>>(part_acc, part_ml, (bf16*)out, N, H, L, nsplit);
  } else {
    cudaFuncSetAttribute(latent_attn_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    latent_attn_kernel<float><<<grid, LAT_WARPS * 32, smem, st>>>((const float*)qlat, (const float*)q, q_stride,
                                                                  (const float*)cache, slot_stride, meta, tok_seq,
                                                                  (float*)out, N, H, D, R, L, scale, nsplit, part_acc,
                                                                  part_ml);
    if (nsplit > 1) latent_combine_kernel<float><<<dim3(N, H), 128, 0, st>>>(part_acc, part_ml, (float*)out, N, H, L, nsplit);
  }
  return (int)cudaGetLastError();
}

int hyb_causal_softmax(const float* s, void* p, long long rows, int rows_per_head, int keys, int first_pos, float scale,
                       int window, int key0, int sink, int split, float cap, const float* sink_vals, int sink_heads,
                       int dt, cudaStream_t st) {
  if (rows == 0) return 0;
  if (scale <= 0.f) return -3;  // the row maximum is taken before scaling
  if (sink_vals && sink_heads < 1) return -2;
  // rows of up to 2048 keys in multiples of 8: 8 keys per thread, so only as many warps as the row needs
  int th = (keys & 7) == 0 && keys <= 2048 ? ((keys / 8 + 31) / 32) * 32 : 256;
  if (th != 256 || ((keys & 7) == 0 && keys <= 2048))
    if (((uintptr_t)s | (uintptr_t)p) & 15) return -4;  // the 16-byte loads and stores of that form
  HYB_DISPATCH(dt, (causal_softmax_kernel<bf16><<<(unsigned)rows, th, 0, st>>>(s, (bf16*)p, rows_per_head, keys, first_pos, scale, window, key0, sink, split, cap, sink_vals, sink_heads)),
               (causal_softmax_kernel<float><<<(unsigned)rows, th, 0, st>>>(s, (float*)p, rows_per_head, keys, first_pos, scale, window, key0, sink, split, cap, sink_vals, sink_heads)));
  return (int)cudaGetLastError();
}

int hyb_conv_silu(const void* x, long long x_stride, const void* w, void* state, void* y, long long y_stride,
                  const int* meta, const int* tok_seq, int N, int nseq, int C, int taps, int dt, cudaStream_t st) {
  if (N == 0) return 0;
  dim3 grid(N, (C + 255) / 256), sgrid(nseq, (C + 255) / 256);
  if (dt == 0) {
    conv_silu_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)x, x_stride, (const bf16*)w, (const bf16*)state,
                                                 (bf16*)y, y_stride, meta, tok_seq, C, taps);
    if (taps > 1) conv_state_kernel<bf16><<<sgrid, 256, 0, st>>>((const bf16*)x, x_stride, (bf16*)state, meta, C, taps);
  } else {
    conv_silu_kernel<float><<<grid, 256, 0, st>>>((const float*)x, x_stride, (const float*)w, (const float*)state,
                                                  (float*)y, y_stride, meta, tok_seq, C, taps);
    if (taps > 1) conv_state_kernel<float><<<sgrid, 256, 0, st>>>((const float*)x, x_stride, (float*)state, meta, C, taps);
  }
  return (int)cudaGetLastError();
}

}  // extern "C"

template <typename T, int R, int ROWS>
static int launch_rec_reg(const RecArgs& a, int nseq, cudaStream_t st) {
  int cpw = 32 / R;
  int threads = (a.V + cpw - 1) / cpw * 32;
  size_t smem = (size_t)a.D * sizeof(float4) + 33 * sizeof(float);
  gated_recurrence_reg_kernel<T, R, ROWS><<<dim3(nseq, a.H), threads, smem, st>>>(a);
  return (int)cudaGetLastError();
}

// lanes per value column for the register kernel: the most that keeps the block within 1024 threads (512 with 32
// rows per lane) and gives every key channel a thread of its own; 0 = the shape does not fit
static int rec_lanes(int D, int V) {
  const int cand[3] = {16, 8, 4};
  for (int c = 0; c < 3; ++c) {
    int R = cand[c], cpw = 32 / R, rows = (D + R - 1) / R;
    int threads = (V + cpw - 1) / cpw * 32;
    int max_rows = R == 4 ? 32 : 16, max_threads = R == 4 ? 512 : 1024;
    if (threads <= max_threads && rows <= max_rows && D <= threads) return R;
  }
  return 0;
}

extern "C" {

// variant: 0 = choose, 1 = shared-memory kernel, 2 = register kernel, 3 = prepare / scan / finish (needs the three
// work buffers: prep [N, H, D] float4, bsig [N, H] float, oraw [N, H * V] float).  "Choose" takes 3 for steps that
// bring more tokens than sequences (prompts) when the buffers are given and D <= 256, else 2 when the shape fits,
// else 1.
int hyb_gated_recurrence(const RecArgs* args, int nseq, int N, int dt, int variant, void* prep, float* bsig,
                         float* oraw, cudaStream_t st) {
  if (nseq == 0) return 0;
  RecArgs a = *args;
  if (a.V > 1024 || a.H % a.G) return -3;
  bool can3 = prep && bsig && oraw && a.D <= 256;
  if (variant == 3 && !can3) return -3;
  if (variant == 3 || (variant == 0 && can3 && N > nseq)) {
    int R = a.D <= 128 ? 8 : 16, cpw = 32 / R;
    int cols = 256 / R;                       // value columns per block at 256 threads
    if (cols > a.V) cols = (a.V + cpw - 1) / cpw * cpw;
    int vs = (a.V + cols - 1) / cols;
    int threads = cols / cpw * 32;
    int need = (a.D + 31) / 32 * 32;          // one staging thread per key channel
    if (threads < need) threads = need;
    size_t smem = 2 * (size_t)a.D * sizeof(float4);
    dim3 g1(N, a.H), g2(nseq, a.H, vs);
    if (dt == 0) {
      rec_prep_kernel<bf16><<<g1, 128, 0, st>>>(a, (float4*)prep, bsig);
      if (R == 8) rec_scan_kernel<bf16, 8><<<g2, threads, smem, st>>>(a, (const float4*)prep, bsig, oraw, cols);
      else rec_scan_kernel<bf16, 16><<<g2, threads, smem, st>>>(a, (const float4*)prep, bsig, oraw, cols);
      rec_finish_kernel<bf16><<<g1, 128, 0, st>>>(a, oraw);
    } else {
      rec_prep_kernel<float><<<g1, 128, 0, st>>>(a, (float4*)prep, bsig);
      if (R == 8) rec_scan_kernel<float, 8><<<g2, threads, smem, st>>>(a, (const float4*)prep, bsig, oraw, cols);
      else rec_scan_kernel<float, 16><<<g2, threads, smem, st>>>(a, (const float4*)prep, bsig, oraw, cols);
      rec_finish_kernel<float><<<g1, 128, 0, st>>>(a, oraw);
    }
    return (int)cudaGetLastError();
  }
  int R = variant != 1 ? rec_lanes(a.D, a.V) : 0;
  if (variant == 2 && R == 0) return -3;
  if (R == 4) return dt == 0 ? launch_rec_reg<bf16, 4, 32>(a, nseq, st) : launch_rec_reg<float, 4, 32>(a, nseq, st);
  if (R == 8) return dt == 0 ? launch_rec_reg<bf16, 8, 16>(a, nseq, st) : launch_rec_reg<float, 8, 16>(a, nseq, st);
  if (R == 16) return dt == 0 ? launch_rec_reg<bf16, 16, 16>(a, nseq, st) : launch_rec_reg<float, 16, 16>(a, nseq, st);
  size_t smem = ((size_t)a.D * a.V + 3 * a.D + 33) * sizeof(float);
  if (smem > 220 * 1024) return -3;
  int threads = (a.V + 31) / 32 * 32;
  dim3 grid(nseq, a.H);
  if (dt == 0) {
    cudaFuncSetAttribute(gated_recurrence_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    gated_recurrence_kernel<bf16><<<grid, threads, smem, st>>>(a);
  } else {
    cudaFuncSetAttribute(gated_recurrence_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    gated_recurrence_kernel<float><<<grid, threads, smem, st>>>(a);
  }
  return (int)cudaGetLastError();
}

#ifndef MDI_BUILD_DIGEST_STR
#define MDI_BUILD_DIGEST_STR "unknown"
#endif
const char* hyb_build_digest() { return "MDI_BUILD_DIGEST:" MDI_BUILD_DIGEST_STR; }

const char* hyb_error_string(int code) { return cudaGetErrorString((cudaError_t)code); }

}  // extern "C"

// =========================================================================================================
// windowed grouped-query attention, per-layer token embedding gate, mixture of experts
// =========================================================================================================
namespace hyb {

__device__ __forceinline__ float gelu_tanhf_(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// One block per token.  Warps walk the H query heads and then the G key heads: rotate the first `nrot` entries
// (entry 2i with 2i+1, angle pos * inv_freq[i]), divide the head by its root mean square over D, store queries
// in place and keys into the slot's cache row; the values are copied behind the keys.  D <= 256.
// qw / kw (optional, [D], shared by the heads) multiply the normalised query / key.  With `lam` the value written is
// (1 - lam) * v + lam * v_first, the blend with another layer's values of the same token, evaluated in fp32.
#define WA_MAXD 8
template <typename T>
__global__ void window_append_kernel(T* __restrict__ q, long long q_stride, const T* __restrict__ k, long long k_stride,
                                     const T* __restrict__ v, long long v_stride, const float* __restrict__ inv_freq,
                                     T* __restrict__ cache, long long slot_stride, const int* __restrict__ meta,
                                     const int* __restrict__ tok_seq, int H, int G, int D, int V, int nrot, float eps,
                                     const T* __restrict__ qw, const T* __restrict__ kw, const T* __restrict__ v_first,
                                     long long vf_stride, const T* __restrict__ lam) {
  int t = blockIdx.x;
  const int* m = meta + 4 * tok_seq[t];
  int pos = m[3] + (t - m[0]);
  T* row = cache + (size_t)m[2] * slot_stride + (size_t)pos * (G * (D + V));
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  float fpos = (float)pos;
  for (int hv = w; hv < H + G; hv += nw) {
    const T* src = hv < H ? q + (size_t)t * q_stride + (size_t)hv * D : k + (size_t)t * k_stride + (size_t)(hv - H) * D;
    T* dst = hv < H ? q + (size_t)t * q_stride + (size_t)hv * D : row + (size_t)(hv - H) * D;
    const T* nw_ = hv < H ? qw : kw;
    float y[WA_MAXD];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < WA_MAXD; ++c) {
      int d = lane + 32 * c;
      y[c] = 0.f;
      if (d < D) {
        float x = to_f(src[d]);
        if (d < nrot) {
          float o = to_f(src[d ^ 1]), sn, cs;
          sincosf(fpos * inv_freq[d >> 1], &sn, &cs);
          x = (d & 1) ? x * cs + o * sn : x * cs - o * sn;
        }
        y[c] = x;
        ss += x * x;
      }
    }
    ss = warp_sum(ss);  // also orders every lane's loads before the in-place stores below
    float inv = 1.f / sqrtf(ss / D + eps);
#pragma unroll
    for (int c = 0; c < WA_MAXD; ++c) {
      int d = lane + 32 * c;
      if (d < D) dst[d] = from_f<T>(nw_ ? y[c] * inv * to_f(nw_[d]) : y[c] * inv);
    }
  }
  const T* vs = v + (size_t)t * v_stride;
  T* vd = row + (size_t)G * D;
  if (lam) {
    float l = to_f(lam[0]);
    const T* vf = v_first + (size_t)t * vf_stride;
    for (int i = threadIdx.x; i < G * V; i += blockDim.x) vd[i] = from_f<T>((1.f - l) * to_f(vs[i]) + l * to_f(vf[i]));
    return;
  }
  for (int i = threadIdx.x; i < G * V; i += blockDim.x) vd[i] = vs[i];
}

// One block per (token, key/value head); warp w is query head g * rep + w.  A tile of 32 cached keys and values is
// staged in shared memory as fp32 once and used by all heads of the group; lane j scores key j, the online softmax
// and the weighted sum are fp32; the result is multiplied by sigmoid(gate) per head.  V <= 256.
// With nsplit > 1 (few tokens: decoding) block z takes every nsplit-th tile and leaves its unnormalised sum, running
// maximum and denominator in part_acc / part_ml; window_combine_kernel merges the shares and applies the gate.
// mask_kind 0: the last `window` positions (0 = all earlier ones); 1: the positions of the token's own block of `window`
// positions, blocks numbered from the first position of the sequence.  sink != 0: a slot of score zero without a value joins the
// softmax denominator.  gate_mode 1: sigmoid(gate[t, h]) per head; 2: sigmoid(gate[t, h * V + d]) per output channel.
// cap > 0: a scaled score s becomes cap * tanh(s / cap).  sink_vals (with sink != 0): the sink's score is sink_vals[h]
// (fp32, neither scaled nor capped) instead of zero.
#define WT_TILE 32
#define WT_MAXV 8
template <typename T>
__global__ void window_attn_kernel(const T* __restrict__ q, long long q_stride, const T* __restrict__ gate,
                                   long long g_stride, const T* __restrict__ cache, long long slot_stride,
                                   const int* __restrict__ meta, const int* __restrict__ tok_seq, T* __restrict__ out,
                                   int H, int G, int D, int V, float scale, int window, int nsplit,
                                   float* __restrict__ part_acc, float* __restrict__ part_ml, int mask_kind, int sink,
                                   int gate_mode, int vec, float cap, const float* __restrict__ sink_vals) {
  extern __shared__ float sm[];
  int rep = H / G;
  float* qs = sm;                       // [rep][D]
  float* Kt = qs + rep * D;             // [32][D + 1]
  float* Vt = Kt + WT_TILE * (D + 1);   // [32][V]
  int t = blockIdx.x, g = blockIdx.y;
  const int* m = meta + 4 * tok_seq[t];
  int pos = m[3] + (t - m[0]);
  int lo = window > 0 ? (mask_kind == 1 ? (pos / window) * window : max(0, pos - window + 1)) : 0;
  const T* base = cache + (size_t)m[2] * slot_stride;
  int rowlen = G * (D + V);
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < rep * D; i += blockDim.x)
    qs[i] = to_f(q[(size_t)t * q_stride + (size_t)g * rep * D + i]);
  float acc[WT_MAXV];
#pragma unroll
  for (int c = 0; c < WT_MAXV; ++c) acc[c] = 0.f;
  float mx = -INFINITY, l = 0.f;
  __syncthreads();
  for (int j0 = lo + (int)blockIdx.z * WT_TILE; j0 <= pos; j0 += WT_TILE * nsplit) {
    __syncthreads();
    if (vec) {
      // 8 values per load, four loads of a thread in flight before the first is used: the tile costs one or two
      // trips to memory instead of one per value
      int dv = D >> 3, vv = V >> 3;
      int nk = WT_TILE * dv, nt = nk + WT_TILE * vv;
      for (int i0 = threadIdx.x; i0 < nt; i0 += 4 * blockDim.x) {
        float f[4][8];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          int i = i0 + u * blockDim.x;
          if (i < nt) {
            bool isk = i < nk;
            int ii = isk ? i : i - nk, per = isk ? dv : vv;
            int j = ii / per, c = ii - j * per;
            if (j0 + j <= pos) {
              load8(base + (size_t)(j0 + j) * rowlen + (isk ? g * D : G * D + g * V) + c * 8, f[u]);
            } else {
#pragma unroll
              for (int e = 0; e < 8; ++e) f[u][e] = 0.f;
            }
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          int i = i0 + u * blockDim.x;
          if (i < nt) {
            bool isk = i < nk;
            int ii = isk ? i : i - nk, per = isk ? dv : vv;
            int j = ii / per, c = ii - j * per;
            float* dst = isk ? Kt + j * (D + 1) + c * 8 : Vt + j * V + c * 8;
#pragma unroll
            for (int e = 0; e < 8; ++e) dst[e] = f[u][e];
          }
        }
      }
    } else {
      for (int i = threadIdx.x; i < WT_TILE * D; i += blockDim.x) {
        int j = i / D, d = i - j * D;
        Kt[j * (D + 1) + d] = j0 + j <= pos ? to_f(base[(size_t)(j0 + j) * rowlen + g * D + d]) : 0.f;
      }
      for (int i = threadIdx.x; i < WT_TILE * V; i += blockDim.x) {
        int j = i / V, d = i - j * V;
        Vt[i] = j0 + j <= pos ? to_f(base[(size_t)(j0 + j) * rowlen + G * D + g * V + d]) : 0.f;
      }
    }
    __syncthreads();
    float s = -INFINITY;
    if (j0 + lane <= pos) {
      const float* qr = qs + w * D;
      const float* kr = Kt + lane * (D + 1);
      float a = 0.f;
      for (int d = 0; d < D; ++d) a += qr[d] * kr[d];
      s = a * scale;
      if (cap > 0.f) s = cap * tanhf(s / cap);
    }
    float mn = fmaxf(mx, warp_max(s));
    float pj = j0 + lane <= pos ? expf(s - mn) : 0.f;
    float corr = expf(mx - mn);  // first tile: exp(-inf) = 0
    l = l * corr + warp_sum(pj);
    mx = mn;
#pragma unroll
    for (int c = 0; c < WT_MAXV; ++c) acc[c] *= corr;
    for (int j = 0; j < WT_TILE; ++j) {
      float pv = __shfl_sync(0xffffffffu, pj, j);
#pragma unroll
      for (int c = 0; c < WT_MAXV; ++c) {
        int d = lane + 32 * c;
        if (d < V) acc[c] += pv * Vt[j * V + d];
      }
    }
  }
  int h = g * rep + w;
  if (nsplit > 1) {
    size_t row = ((size_t)blockIdx.z * gridDim.x + t) * H + h;
#pragma unroll
    for (int c = 0; c < WT_MAXV; ++c) {
      int d = lane + 32 * c;
      if (d < V) part_acc[row * V + d] = acc[c];
    }
    if (lane == 0) { part_ml[2 * row] = mx; part_ml[2 * row + 1] = l; }
    return;
  }
  if (sink) {  // the slot without a value: shift to max(mx, its score), add its weight to the denominator
    float sv = sink_vals ? sink_vals[h] : 0.f;
    float mn = fmaxf(mx, sv), corr = expf(mx - mn);
    l = l * corr + expf(sv - mn);
#pragma unroll
    for (int c = 0; c < WT_MAXV; ++c) acc[c] *= corr;
  }
  float gt = gate && gate_mode == 1 ? sigmoidf_(to_f(gate[(size_t)t * g_stride + h])) : 1.f;
  float inv = gt / l;
#pragma unroll
  for (int c = 0; c < WT_MAXV; ++c) {
    int d = lane + 32 * c;
    if (d < V) {
      float o = acc[c] * inv;
      if (gate && gate_mode == 2) o *= sigmoidf_(to_f(gate[(size_t)t * g_stride + (size_t)h * V + d]));
      out[(size_t)t * H * V + (size_t)h * V + d] = from_f<T>(o);
    }
  }
}

// Merge of the key shares of window_attn_kernel: one warp per (token, head), nsplit <= 32.  Lane s reads share s's
// running maximum and denominator (one round of loads instead of a chain of nsplit), the weights exp(m_s - M) are
// handed round by shuffles while lane d sums channel d over the shares.
template <typename T>
__global__ void window_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                      const T* __restrict__ gate, long long g_stride, T* __restrict__ out, int N, int H,
                                      int V, int nsplit, int sink, int gate_mode, const float* __restrict__ sink_vals) {
  int t = blockIdx.x, h = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (h >= H) return;
  float ms = -INFINITY, ls = 0.f;
  if (lane < nsplit) {
    const float* ml = part_ml + 2 * (((size_t)lane * N + t) * H + h);
    ms = ml[0];
    ls = ml[1];
  }
  float M = warp_max(ms);
  float sv = sink && sink_vals ? sink_vals[h] : 0.f;
  if (sink) M = fmaxf(M, sv);
  float ws = lane < nsplit ? expf(ms - M) : 0.f;  // a share without keys: exp(-inf) = 0
  float l = warp_sum(ls * ws) + (sink ? expf(sv - M) : 0.f);
  float gt = gate && gate_mode == 1 ? sigmoidf_(to_f(gate[(size_t)t * g_stride + h])) : 1.f;
  if ((V & 3) == 0) {  // four channels per lane, eight shares' loads in flight: the merge is a chain of round trips
    for (int d0 = 0; d0 < V; d0 += 128) {
      int d = d0 + 4 * lane;
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
      for (int s = 0; s < nsplit; ++s) {
        float w = __shfl_sync(0xffffffffu, ws, s);
        if (d < V) {
          float4 x = *reinterpret_cast<const float4*>(part_acc + ((((size_t)s * N + t) * H + h)) * V + d);
          a.x += x.x * w; a.y += x.y * w; a.z += x.z * w; a.w += x.w * w;
        }
      }
      if (d < V) {
        float o[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = o[e] * gt / l;
          if (gate && gate_mode == 2) v *= sigmoidf_(to_f(gate[(size_t)t * g_stride + (size_t)h * V + d + e]));
          out[(size_t)t * H * V + (size_t)h * V + d + e] = from_f<T>(v);
        }
      }
    }
    return;
  }
  for (int d0 = 0; d0 < V; d0 += 32) {
    int d = d0 + lane;
    float a = 0.f;
#pragma unroll 4
    for (int s = 0; s < nsplit; ++s) {
      float w = __shfl_sync(0xffffffffu, ws, s);
      if (d < V) a += part_acc[((((size_t)s * N + t) * H + h)) * V + d] * w;
    }
    if (d < V) {
      float o = a * gt / l;
      if (gate && gate_mode == 2) o *= sigmoidf_(to_f(gate[(size_t)t * g_stride + (size_t)h * V + d]));
      out[(size_t)t * H * V + (size_t)h * V + d] = from_f<T>(o);
    }
  }
}

// out[r, h*hv + d] = a[h, r, d] * sigmoid(g[r, h]): one gate per head, a stored head-major.
template <typename T>
__global__ void head_gate_kernel(const T* __restrict__ a, const T* __restrict__ g, long long g_stride,
                                 T* __restrict__ out, int rows, int heads, int hv) {
  int r = blockIdx.x;
  int n = heads * hv;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    int h = c / hv, d = c - h * hv;
    float v = to_f(a[((size_t)h * rows + r) * hv + d]);
    out[(size_t)r * n + c] = from_f<T>(v * sigmoidf_(to_f(g[(size_t)r * g_stride + h])));
  }
}

// out[r, c] = gelu_tanh(z[r, c]) * table[tokens[r], col0 + c]
template <typename T>
__global__ void token_side_gate_kernel(const T* __restrict__ z, long long z_stride, const T* __restrict__ table,
                                       long long t_stride, int col0, const int* __restrict__ tokens,
                                       T* __restrict__ out, int d) {
  int r = blockIdx.x;
  const T* e = table + (size_t)tokens[r] * t_stride + col0;
  for (int c = threadIdx.x; c < d; c += blockDim.x)
    out[(size_t)r * d + c] = from_f<T>(gelu_tanhf_(to_f(z[(size_t)r * z_stride + c])) * to_f(e[c]));
}

// One thread per token: the `top` largest logits (ties to the lower index).  mode 0: scores = sigmoid(logit), each
// on its own; mode 1: scores = softmax restricted to the selected logits; mode 2: scores s = softmax over ALL E logits,
// the choice goes by s + correction (correction: E floats, optional), the weights are the chosen s divided by their
// sum + 1e-20.
__global__ void router_topk_kernel(const float* __restrict__ z, int* __restrict__ idx, float* __restrict__ wt, int N,
                                   int E, int top, int mode, const float* __restrict__ correction) {
  int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= N) return;
  const float* row = z + (size_t)t * E;
  if (mode == 2) {
    float m = -INFINITY, den = 0.f;
    for (int e = 0; e < E; ++e) m = fmaxf(m, row[e]);
    for (int e = 0; e < E; ++e) den += expf(row[e] - m);
    float tot = 0.f;
    for (int k = 0; k < top; ++k) {
      int best = -1;
      float bv = -INFINITY, bs = 0.f;
      for (int e = 0; e < E; ++e) {
        bool taken = false;
        for (int j = 0; j < k; ++j) taken |= idx[(size_t)t * top + j] == e;
        float sc = expf(row[e] - m) / den;
        float v = correction ? sc + correction[e] : sc;
        if (!taken && (best < 0 || v > bv)) { best = e; bv = v; bs = sc; }
      }
      idx[(size_t)t * top + k] = best;
      wt[(size_t)t * top + k] = bs;
      tot += bs;
    }
    tot += 1e-20f;
    for (int k = 0; k < top; ++k) wt[(size_t)t * top + k] /= tot;
    return;
  }
  for (int k = 0; k < top; ++k) {
    int best = -1;
    float bv = -INFINITY;
    for (int e = 0; e < E; ++e) {
      bool taken = false;
      for (int j = 0; j < k; ++j) taken |= idx[(size_t)t * top + j] == e;
      float v = row[e];
      if (!taken && (best < 0 || v > bv)) { best = e; bv = v; }
    }
    idx[(size_t)t * top + k] = best;
    wt[(size_t)t * top + k] = mode == 0 ? sigmoidf_(bv) : bv;
  }
  if (mode == 1) {  // the first choice holds the largest logit
    float* w = wt + (size_t)t * top;
    float m = w[0], sum = 0.f;
    for (int k = 0; k < top; ++k) { w[k] = expf(w[k] - m); sum += w[k]; }
    for (int k = 0; k < top; ++k) w[k] /= sum;
  }
}

template <typename T>
__device__ __forceinline__ float dot_row(const T* __restrict__ wrow, const float* __restrict__ xs, int n, int lane) {
  float a = 0.f;
  if ((n & 7) == 0) {
    for (int c = lane * 8; c < n; c += 256) {
      float f[8];
      load8(wrow + c, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) a += f[i] * xs[c + i];
    }
  } else {
    for (int c = lane; c < n; c += 32) a += to_f(wrow[c]) * xs[c];
  }
  return warp_sum(a);
}

// Experts by index for few tokens.  A pair p = (token, choice k) names expert idx[p] and score wt[p].  One block owns
// 32 output rows of ONE expert and serves every pair that chose it, MOE_PCH pairs at a time, so an expert's weights
// cross the memory system once however many pairs share it; experts nobody chose cost one scan of idx.
//   MODE 0 (up):   y[p, f] = relu(w[e][f, :] . round_T(wt[p] * x[p / top, :]))^2     x in T, K = width
//   MODE 1 (down): y[p, c] = w[e][c, :] . a[p, :]                                    a fp32, K = ff
//   MODE 2 (gated up): y[p, f] = silu(w[e][f, :] . x) * (w[e][R + f, :] . x), x = x[p / top, :] unscaled; an expert's
//                  matrix is [2R, K], its gate rows first and its up rows behind them
//                  glu 0: silu(g) * u as above; glu 1 (clamped): g' = min(g, limit), u' = clamp(u, -limit, limit),
//                  y = g' * sigmoid(1.702 g') * (u' + 1)
// A pair whose index is not below the grid's expert count (an identity expert: no tensors) is served by no block.
#define MOE_ROWS 32
#define MOE_PCH 4
__device__ __forceinline__ float glu_act(float g, float u, int glu, float limit) {
  if (glu == 0) return siluf_(g) * u;
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g * sigmoidf_(1.702f * g) * (u + 1.f);
}
template <typename T, int MODE>
__global__ void moe_pairs_kernel(const void* __restrict__ xin, long long x_stride, const int* __restrict__ idx,
                                 const float* __restrict__ wt, const T* __restrict__ w, float* __restrict__ y, int P,
                                 int top, int K, int R, int pch, int glu, float limit) {
  extern __shared__ float sm[];  // [pch][K]
  __shared__ int match[MOE_PCH];
  __shared__ int s_cnt, s_next;
  int e = blockIdx.x;
  int lane = threadIdx.x & 31, wp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const T* we = w + (size_t)e * (MODE == 2 ? 2 : 1) * R * K;
  if (threadIdx.x == 0) s_next = 0;
  __syncthreads();
  while (true) {
    if (threadIdx.x == 0) {
      int c = 0, p = s_next;
      for (; p < P && c < pch; ++p)
        if (idx[p] == e) match[c++] = p;
      s_cnt = c;
      s_next = p;
    }
    __syncthreads();
    int cnt = s_cnt;
    if (cnt == 0) return;
    for (int m = 0; m < cnt; ++m) {
      int p = match[m];
      if (MODE == 0) {
        const T* x = (const T*)xin + (size_t)(p / top) * x_stride;
        float sc = wt[p];
        for (int c = threadIdx.x; c < K; c += blockDim.x) sm[m * K + c] = to_f(from_f<T>(sc * to_f(x[c])));
      } else if (MODE == 2) {
        const T* x = (const T*)xin + (size_t)(p / top) * x_stride;
        for (int c = threadIdx.x; c < K; c += blockDim.x) sm[m * K + c] = to_f(x[c]);
      } else {
        const float* x = (const float*)xin + (size_t)p * x_stride;
        for (int c = threadIdx.x; c < K; c += blockDim.x) sm[m * K + c] = x[c];
      }
    }
    __syncthreads();
    for (int r = wp; r < MOE_ROWS; r += nw) {
      int f = blockIdx.y * MOE_ROWS + r;
      if (f >= R) break;
      const T* wrow = we + (size_t)f * K;
      float acc[MOE_PCH], first[MOE_PCH];
#pragma unroll
      for (int m = 0; m < MOE_PCH; ++m) first[m] = 0.f;
      for (int half = 0; half < (MODE == 2 ? 2 : 1); ++half) {
      if (half == 1) {
        wrow += (size_t)R * K;
#pragma unroll
        for (int m = 0; m < MOE_PCH; ++m) first[m] = acc[m];
      }
#pragma unroll
      for (int m = 0; m < MOE_PCH; ++m) acc[m] = 0.f;
      if ((K & 7) == 0) {
        // four 16-byte weight loads in flight per lane before any of them is used
        for (int c0 = lane * 8; c0 < K; c0 += 1024) {
          float wv[4][8];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (c0 + 256 * u < K) load8(wrow + c0 + 256 * u, wv[u]);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            int c = c0 + 256 * u;
            if (c < K) {
#pragma unroll
              for (int m = 0; m < MOE_PCH; ++m)
                if (m < cnt) {  // two 16-byte shared loads per lane: no bank conflicts
                  const float4* xv = reinterpret_cast<const float4*>(sm + (size_t)m * K + c);
                  float4 x0 = xv[0], x1 = xv[1];
                  acc[m] += wv[u][0] * x0.x + wv[u][1] * x0.y + wv[u][2] * x0.z + wv[u][3] * x0.w + wv[u][4] * x1.x +
                            wv[u][5] * x1.y + wv[u][6] * x1.z + wv[u][7] * x1.w;
                }
            }
          }
        }
      } else {
        for (int c = lane; c < K; c += 32) {
          float wv = to_f(wrow[c]);
#pragma unroll
          for (int m = 0; m < MOE_PCH; ++m)
            if (m < cnt) acc[m] += wv * sm[m * K + c];
        }
      }
      }
#pragma unroll
      for (int m = 0; m < MOE_PCH; ++m) {
        if (m < cnt) {
          float v = warp_sum(acc[m]);
          float g = MODE == 2 ? warp_sum(first[m]) : 0.f;
          if (lane == 0) {
            if (MODE == 0) { v = fmaxf(v, 0.f); v = v * v; }
            if (MODE == 2) v = glu_act(g, v, glu, limit);
            y[(size_t)match[m] * R + f] = v;
          }
        }
      }
    }
    __syncthreads();
  }
}

// The same work for bf16 weights with K a multiple of 8, streamed: the block's slab of weight rows (32 rows; with a
// gate, the 32 gate rows and the 32 up rows) crosses shared memory in chunks of KC columns through a ring of
// MS_STAGES 16 KB stages filled by 16-byte asynchronous copies, three chunks in flight while one is used, so the
// bytes in flight per SM do not depend on how many warps wait.  A warp owns rows w, w+8, w+16, w+24 of the slab and
// keeps their sums for up to MOE_PCH pairs; a lane takes 8 columns of a chunk (with a gate: lanes 0-15 the gate row,
// lanes 16-31 the up row of the same output).
#define MS_STAGES 4
#define MS_STAGE_ELEMS 8192
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

template <int MODE>
__global__ void __launch_bounds__(256) moe_pairs_stream_kernel(const void* __restrict__ xin, long long x_stride,
                                                               const int* __restrict__ idx, const float* __restrict__ wt,
                                                               const bf16* __restrict__ w, float* __restrict__ y, int P,
                                                               int top, int K, int R, int pch, int glu, float limit) {
  constexpr int KC = MODE == 2 ? 128 : 256;  // columns per chunk
  constexpr int LPR = KC / 8;                // lanes per row of a chunk
  extern __shared__ __align__(16) unsigned char ms_raw[];
  float* xs = reinterpret_cast<float*>(ms_raw);                          // [pch][K]
  bf16* ring = reinterpret_cast<bf16*>(ms_raw + (size_t)pch * K * 4);    // [MS_STAGES][rows][KC]
  __shared__ int match[MOE_PCH];
  __shared__ int s_cnt, s_next;
  int e = blockIdx.x, f0 = blockIdx.y * MOE_ROWS;
  int lane = threadIdx.x & 31, wp = threadIdx.x >> 5;
  const bf16* we = w + (size_t)e * (MODE == 2 ? 2 : 1) * R * K;
  int nchunks = (K + KC - 1) / KC;
  if (threadIdx.x == 0) s_next = 0;
  __syncthreads();
  while (true) {
    if (threadIdx.x == 0) {
      int c = 0, p = s_next;
      for (; p < P && c < pch; ++p)
        if (idx[p] == e) match[c++] = p;
      s_cnt = c;
      s_next = p;
    }
    __syncthreads();
    int cnt = s_cnt;
    if (cnt == 0) return;
    // fill one stage: 1024 vectors of 8 weights, four per thread; rows past R and columns past K become zeros
    auto issue = [&](int kc, int stage) {
      bf16* st = ring + (size_t)stage * MS_STAGE_ELEMS;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        int v = threadIdx.x + 256 * u;
        int sr = v / LPR, cv = v - sr * LPR;
        int f = f0 + (sr & (MOE_ROWS - 1)), k = kc * KC + cv * 8;
        bf16* dst = st + sr * KC + cv * 8;
        if (f < R && k < K) {
          size_t row = MODE == 2 && sr >= MOE_ROWS ? (size_t)R + f : (size_t)f;
          cp_async16(dst, we + row * K + k);
        } else {
          *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
    };
#pragma unroll
    for (int s = 0; s < MS_STAGES - 1; ++s) {
      if (s < nchunks) issue(s, s);
      cp_async_commit();
    }
    for (int m = 0; m < cnt; ++m) {  // the pairs' inputs, while the first chunks travel
      int p = match[m];
      if (MODE == 0) {
        const bf16* x = (const bf16*)xin + (size_t)(p / top) * x_stride;
        float sc = wt[p];
        for (int c = threadIdx.x; c < K; c += blockDim.x) xs[m * K + c] = to_f(from_f<bf16>(sc * to_f(x[c])));
      } else if (MODE == 2) {
        const bf16* x = (const bf16*)xin + (size_t)(p / top) * x_stride;
        for (int c = threadIdx.x; c < K; c += blockDim.x) xs[m * K + c] = to_f(x[c]);
      } else {
        const float* x = (const float*)xin + (size_t)p * x_stride;
        for (int c = threadIdx.x; c < K; c += blockDim.x) xs[m * K + c] = x[c];
      }
    }
    float acc[4][MOE_PCH];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int m = 0; m < MOE_PCH; ++m) acc[i][m] = 0.f;
    int half = MODE == 2 ? lane >> 4 : 0, hl = MODE == 2 ? lane & 15 : lane;
    for (int kc = 0; kc < nchunks; ++kc) {
      cp_async_wait<MS_STAGES - 2>();  // this thread's copies of chunk kc have landed
      __syncthreads();                 // everybody's have, and everybody is done with chunk kc - 1
      int nk = kc + MS_STAGES - 1;
      if (nk < nchunks) issue(nk, nk % MS_STAGES);  // into the stage chunk kc - 1 occupied
      cp_async_commit();
      const bf16* st = ring + (size_t)(kc % MS_STAGES) * MS_STAGE_ELEMS;
      int k = kc * KC + hl * 8;
      if (k < K) {
        float wv[4][8];
#pragma unroll
        for (int i = 0; i < 4; ++i) load8(st + (half * MOE_ROWS + wp + 8 * i) * KC + hl * 8, wv[i]);
#pragma unroll
        for (int m = 0; m < MOE_PCH; ++m)
          if (m < cnt) {
            const float4* xv = reinterpret_cast<const float4*>(xs + (size_t)m * K + k);
            float4 x0 = xv[0], x1 = xv[1];
#pragma unroll
            for (int i = 0; i < 4; ++i)
              acc[i][m] += wv[i][0] * x0.x + wv[i][1] * x0.y + wv[i][2] * x0.z + wv[i][3] * x0.w + wv[i][4] * x1.x +
                           wv[i][5] * x1.y + wv[i][6] * x1.z + wv[i][7] * x1.w;
          }
      }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int f = f0 + wp + 8 * i;
#pragma unroll
      for (int m = 0; m < MOE_PCH; ++m) {
        if (m < cnt) {  // cnt is the same for the whole block: the shuffles below are not divergent
          float v = acc[i][m];
          if (MODE == 2) {
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            float g = __shfl_sync(0xffffffffu, v, 0), u = __shfl_sync(0xffffffffu, v, 16);
            v = glu_act(g, u, glu, limit);
          } else {
            v = warp_sum(v);
            if (MODE == 0) { v = fmaxf(v, 0.f); v = v * v; }
          }
          if (lane == 0 && f < R) y[(size_t)match[m] * R + f] = v;
        }
      }
    }
    __syncthreads();
  }
}

// out[t, c] = sum_k wt[t * top + k] * y[t * top + k, c] (wt absent: plain sum), summed in the order of k.  With `idx`,
// a choice whose index is E or more is an identity expert: its term is wt * h[t, c], the token's own input row.
template <typename T>
__global__ void moe_sum_kernel(const float* __restrict__ y, const float* __restrict__ wt, T* __restrict__ out, int top,
                               int C, const int* __restrict__ idx, int E, const T* __restrict__ h, long long h_stride) {
  int t = blockIdx.x;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float a = 0.f;
    for (int k = 0; k < top; ++k) {
      size_t p = (size_t)t * top + k;
      float term = idx && idx[p] >= E ? to_f(h[(size_t)t * h_stride + c]) : y[p * C + c];
      a += (wt ? wt[p] : 1.f) * term;
    }
    out[(size_t)t * C + c] = from_f<T>(a);
  }
}

template <typename T>
__global__ void gather_scale_rows_kernel(const T* __restrict__ h, long long h_stride, const int* __restrict__ rows,
                                         const float* __restrict__ scale, T* __restrict__ out, int C) {
  int i = blockIdx.x;
  const T* src = h + (size_t)rows[i] * h_stride;
  if (!scale) {
    for (int c = threadIdx.x; c < C; c += blockDim.x) out[(size_t)i * C + c] = src[c];
    return;
  }
  float w = scale[i];
  for (int c = threadIdx.x; c < C; c += blockDim.x) out[(size_t)i * C + c] = from_f<T>(w * to_f(src[c]));
}

// With `idx`, a choice whose index is E or more is an identity expert: its term is wt * h[t, c] and its row of y is
// not read.
template <typename T>
__global__ void combine_rows_kernel(const T* __restrict__ y, const int* __restrict__ where, const float* __restrict__ wt,
                                    T* __restrict__ out, int top, int C, const int* __restrict__ idx, int E,
                                    const T* __restrict__ h, long long h_stride) {
  int t = blockIdx.x;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float a = 0.f;
    for (int k = 0; k < top; ++k) {
      size_t p = (size_t)t * top + k;
      float term = idx && idx[p] >= E ? to_f(h[(size_t)t * h_stride + c]) : to_f(y[(size_t)where[p] * C + c]);
      a += (wt ? wt[p] : 1.f) * term;
    }
    out[(size_t)t * C + c] = from_f<T>(a);
  }
}

// out[r, f] = act(in[r, f]) * in[r, F + f]: the product of a gated feed-forward whose gate and up projections are
// the two halves of one row.  act 0: silu, 1: gelu (tanh form), 2: the clamped form of glu_act with `limit`.
__device__ __forceinline__ float act_mul_one(float g, float u, int act, float limit) {
  return act == 2 ? glu_act(g, u, 1, limit) : (act == 0 ? siluf_(g) : gelu_tanhf_(g)) * u;
}
template <typename T>
__global__ void act_mul_rows_kernel(const T* __restrict__ in, long long in_stride, T* __restrict__ out, int F, int act,
                                    long long total, float limit) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  long long r = i / F;
  int f = (int)(i - r * F);
  const T* row = in + (size_t)r * in_stride;
  float g = to_f(row[f]), u = to_f(row[F + f]);
  out[i] = from_f<T>(act_mul_one(g, u, act, limit));
}

// The same, 8 values per thread with 16-byte loads and stores (F and the row stride multiples of 8, bases aligned).
template <typename T>
__global__ void act_mul_rows_vec_kernel(const T* __restrict__ in, long long in_stride, T* __restrict__ out, int F, int act,
                                        long long total8, float limit) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total8) return;
  int f8 = F >> 3;
  long long r = i / f8;
  int c = (int)(i - r * f8) * 8;
  const T* row = in + (size_t)r * in_stride;
  float g[8], u[8];
  load8(row + c, g);
  load8(row + F + c, u);
#pragma unroll
  for (int e = 0; e < 8; ++e) g[e] = act_mul_one(g[e], u[e], act, limit);
  store8(out + (size_t)r * F + c, g);
}

// x[r, c] += ls1[c] * a[r, c] + ls2[c] * (b[r, c] + b2[r, c]): the residual update of a block whose mixer and
// feed-forward read the same normed input, each branch with a learned scale per channel.  b, b2 and the scales are
// optional (absent scale = 1); x is the fp32 residual.
template <typename T>
__global__ void scaled_branches_kernel(float* __restrict__ x, long long x_stride, const T* __restrict__ a,
                                       long long a_stride, const T* __restrict__ ls1, const T* __restrict__ b,
                                       long long b_stride, const T* __restrict__ b2, long long b2_stride,
                                       const T* __restrict__ ls2, int C) {
  size_t r = blockIdx.x;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float y = to_f(a[r * a_stride + c]) * (ls1 ? to_f(ls1[c]) : 1.f);
    if (b) {
      float f = to_f(b[r * b_stride + c]);
      if (b2) f += to_f(b2[r * b2_stride + c]);
      y += f * (ls2 ? to_f(ls2[c]) : 1.f);
    }
    x[r * x_stride + c] += y;
  }
}

}  // namespace hyb

extern "C" {

int hyb_window_append(void* q, long long q_stride, const void* k, long long k_stride, const void* v, long long v_stride,
                      const float* inv_freq, void* cache, long long slot_stride, const int* meta, const int* tok_seq,
                      int N, int H, int G, int D, int V, int nrot, float eps, const void* qw, const void* kw,
                      const void* v_first, long long vf_stride, const void* lam, int dt, cudaStream_t st) {
  if (N == 0) return 0;
  if (D > 32 * WA_MAXD || nrot > D || (nrot & 1) || (nrot > 0 && !inv_freq)) return -3;
  if (lam && !v_first) return -2;
  HYB_DISPATCH(dt,
               (window_append_kernel<bf16><<<N, 128, 0, st>>>((bf16*)q, q_stride, (const bf16*)k, k_stride, (const bf16*)v,
                                                              v_stride, inv_freq, (bf16*)cache, slot_stride, meta, tok_seq,
                                                              H, G, D, V, nrot, eps, (const bf16*)qw, (const bf16*)kw,
                                                              (const bf16*)v_first, vf_stride, (const bf16*)lam)),
               (window_append_kernel<float><<<N, 128, 0, st>>>((float*)q, q_stride, (const float*)k, k_stride,
                                                               (const float*)v, v_stride, inv_freq, (float*)cache,
                                                               slot_stride, meta, tok_seq, H, G, D, V, nrot, eps,
                                                               (const float*)qw, (const float*)kw, (const float*)v_first,
                                                               vf_stride, (const float*)lam)));
  return (int)cudaGetLastError();
}

int hyb_window_attn(const void* q, long long q_stride, const void* gate, long long g_stride, const void* cache,
                    long long slot_stride, const int* meta, const int* tok_seq, void* out, int N, int H, int G, int D,
                    int V, float scale, int window, int nsplit, float* part_acc, float* part_ml, int mask_kind, int sink,
                    int gate_mode, float cap, const float* sink_vals, int dt, cudaStream_t st) {
  if (N == 0) return 0;
  if (mask_kind < 0 || mask_kind > 1 || (mask_kind == 1 && window < 1) || gate_mode < 0 || gate_mode > 2) return -3;
  int rep = G > 0 ? H / G : 0;
  if (rep < 1 || rep * G != H || rep > 32 || V > 32 * WT_MAXV) return -3;
  if (nsplit < 1 || (nsplit > 1 && (!part_acc || !part_ml))) return -2;
  size_t smem = ((size_t)rep * D + (size_t)WT_TILE * (D + 1) + (size_t)WT_TILE * V) * sizeof(float);
  if (smem > 220 * 1024) return -3;
  if (nsplit > 32) return -3;  // the merge gives each key share a lane
  dim3 grid(N, G, nsplit), cgrid(N, (H + 3) / 4);
  // 16-byte loads of cache rows: every head's slice of every row starts on a 16-byte (fp32: 32-byte) boundary
  int vec = D % 8 == 0 && V % 8 == 0 && slot_stride % 8 == 0 && (uintptr_t)cache % 32 == 0;
  cudaError_t e;
  if (dt == 0) {
    if (smem > 48 * 1024 && (e = cudaFuncSetAttribute(window_attn_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return (int)e;
    window_attn_kernel<bf16><<<grid, 32 * rep, smem, st>>>((const bf16*)q, q_stride, (const bf16*)gate, g_stride,
                                                           (const bf16*)cache, slot_stride, meta, tok_seq, (bf16*)out, H,
                                                           G, D, V, scale, window, nsplit, part_acc, part_ml, mask_kind, sink,
                                                           gate_mode, vec, cap, sink_vals);
    if (nsplit > 1)
      window_combine_kernel<bf16><<<cgrid, 128, 0, st>>>(part_acc, part_ml, (const bf16*)gate, g_stride, (bf16*)out, N, H, V, nsplit, sink, gate_mode, sink_vals);
  } else {
    if (smem > 48 * 1024 && (e = cudaFuncSetAttribute(window_attn_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return (int)e;
    window_attn_kernel<float><<<grid, 32 * rep, smem, st>>>((const float*)q, q_stride, (const float*)gate, g_stride,
                                                            (const float*)cache, slot_stride, meta, tok_seq, (float*)out,
                                                            H, G, D, V, scale, window, nsplit, part_acc, part_ml, mask_kind, sink,
                                                            gate_mode, vec, cap, sink_vals);
    if (nsplit > 1)
      window_combine_kernel<float><<<cgrid, 128, 0, st>>>(part_acc, part_ml, (const float*)gate, g_stride, (float*)out, N, H, V, nsplit, sink, gate_mode, sink_vals);
  }
  return (int)cudaGetLastError();
}

int hyb_head_gate(const void* a, const void* g, long long g_stride, void* out, int rows, int heads, int hv, int dt,
                  cudaStream_t st) {
  if (rows == 0) return 0;
  HYB_DISPATCH(dt,
               (head_gate_kernel<bf16><<<rows, 256, 0, st>>>((const bf16*)a, (const bf16*)g, g_stride, (bf16*)out, rows,
                                                             heads, hv)),
               (head_gate_kernel<float><<<rows, 256, 0, st>>>((const float*)a, (const float*)g, g_stride, (float*)out,
                                                              rows, heads, hv)));
  return (int)cudaGetLastError();
}

int hyb_token_side_gate(const void* z, long long z_stride, const void* table, long long t_stride, int col0,
                        const int* tokens, void* out, int N, int d, int dt, cudaStream_t st) {
  if (N == 0) return 0;
  int th = d >= 256 ? 256 : (d >= 64 ? 64 : 32);
  HYB_DISPATCH(dt,
               (token_side_gate_kernel<bf16><<<N, th, 0, st>>>((const bf16*)z, z_stride, (const bf16*)table, t_stride,
                                                               col0, tokens, (bf16*)out, d)),
               (token_side_gate_kernel<float><<<N, th, 0, st>>>((const float*)z, z_stride, (const float*)table, t_stride,
                                                                col0, tokens, (float*)out, d)));
  return (int)cudaGetLastError();
}

int hyb_router_topk(const float* z, int* idx, float* wt, int N, int E, int top, int mode, const float* correction,
                    cudaStream_t st) {
  if (N == 0) return 0;
  if (top < 1 || top > E || mode < 0 || mode > 2) return -3;
  router_topk_kernel<<<(N + 63) / 64, 64, 0, st>>>(z, idx, wt, N, E, top, mode, correction);
  return (int)cudaGetLastError();
}

}  // extern "C"

template <typename T, int MODE>
static int launch_moe_pairs(const void* x, long long x_stride, const int* idx, const float* wt, const void* w, float* y,
                            int P, int top, int K, int R, int E, cudaStream_t st, int glu = 0, float limit = 0.f) {
  // shared memory only for the pairs there can be, and at most 64 KB while more than one pair is staged: three
  // blocks per SM keep more weight loads in flight than one block that serves four pairs at once
  int pch = P < MOE_PCH ? P : MOE_PCH;
  if constexpr (sizeof(T) == 2) {
    if (K % 8 == 0 && (uintptr_t)w % 16 == 0) {  // streamed form: 64 KB of stages beside at most 32 KB of inputs
      int spch = pch;
      while (spch > 1 && (size_t)spch * K * sizeof(float) > 32 * 1024) --spch;
      size_t ssm = (size_t)spch * K * sizeof(float) + (size_t)MS_STAGES * MS_STAGE_ELEMS * sizeof(bf16);
      if (ssm <= 200 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(moe_pairs_stream_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ssm);
        if (e != cudaSuccess) return (int)e;
        dim3 sgrid(E, (R + MOE_ROWS - 1) / MOE_ROWS);
        moe_pairs_stream_kernel<MODE><<<sgrid, 256, ssm, st>>>(x, x_stride, idx, wt, (const bf16*)w, y, P, top, K, R, spch, glu, limit);
        return (int)cudaGetLastError();
      }
    }
  }
  while (pch > 1 && (size_t)pch * K * sizeof(float) > 64 * 1024) --pch;
  size_t smem = (size_t)pch * K * sizeof(float);
  if (smem > 200 * 1024) return -3;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(moe_pairs_kernel<T, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(E, (R + MOE_ROWS - 1) / MOE_ROWS);
  moe_pairs_kernel<T, MODE><<<grid, 256, smem, st>>>(x, x_stride, idx, wt, (const T*)w, y, P, top, K, R, pch, glu, limit);
  return (int)cudaGetLastError();
}

extern "C" {

// act [N*top, ff] fp32.  gated 0: squared-ReLU of the chosen experts' up projections of the score-weighted token
// (up [E, ff, C]).  gated 1: silu(gate x) * (up x) of the token as it is (up [E, 2 ff, C], gate rows first).
// gated 2: the clamped form (glu_act) with `limit`.
int hyb_moe_up(const void* h, long long h_stride, const int* idx, const float* wt, const void* up, float* act, int N,
               int top, int C, int ff, int E, int gated, float limit, int dt, cudaStream_t st) {
  if (N == 0) return 0;
  if (gated < 0 || gated > 2) return -3;
  if (gated) {
    if (dt == 0) return launch_moe_pairs<bf16, 2>(h, h_stride, idx, wt, up, act, N * top, top, C, ff, E, st, gated - 1, limit);
    return launch_moe_pairs<float, 2>(h, h_stride, idx, wt, up, act, N * top, top, C, ff, E, st, gated - 1, limit);
  }
  if (!wt) return -2;
  if (dt == 0) return launch_moe_pairs<bf16, 0>(h, h_stride, idx, wt, up, act, N * top, top, C, ff, E, st);
  return launch_moe_pairs<float, 0>(h, h_stride, idx, wt, up, act, N * top, top, C, ff, E, st);
}

// out [N, C] = sum over a token's choices of the expert's down projection of act, each times wt[choice] when wt is
// given; ypair [N*top, C] fp32 is scratch.  With h, a choice of index >= E adds wt * h[token] (an identity expert).
int hyb_moe_down(const float* act, const int* idx, const float* wt, const void* down, float* ypair, void* out, int N,
                 int top, int C, int ff, int E, const void* h, long long h_stride, int dt, cudaStream_t st) {
  if (N == 0) return 0;
  int rc = dt == 0 ? launch_moe_pairs<bf16, 1>(act, ff, idx, nullptr, down, ypair, N * top, top, ff, C, E, st)
                   : launch_moe_pairs<float, 1>(act, ff, idx, nullptr, down, ypair, N * top, top, ff, C, E, st);
  if (rc) return rc;
  const int* ix = h ? idx : nullptr;
  HYB_DISPATCH(dt, (moe_sum_kernel<bf16><<<N, 256, 0, st>>>(ypair, wt, (bf16*)out, top, C, ix, E, (const bf16*)h, h_stride)),
               (moe_sum_kernel<float><<<N, 256, 0, st>>>(ypair, wt, (float*)out, top, C, ix, E, (const float*)h, h_stride)));
  return (int)cudaGetLastError();
}

int hyb_gather_scale_rows(const void* h, long long h_stride, const int* rows, const float* scale, void* out, int M, int C,
                          int dt, cudaStream_t st) {
  if (M == 0) return 0;
  HYB_DISPATCH(dt,
               (gather_scale_rows_kernel<bf16><<<M, 256, 0, st>>>((const bf16*)h, h_stride, rows, scale, (bf16*)out, C)),
               (gather_scale_rows_kernel<float><<<M, 256, 0, st>>>((const float*)h, h_stride, rows, scale, (float*)out, C)));
  return (int)cudaGetLastError();
}

int hyb_combine_rows(const void* y, const int* where, const float* wt, void* out, int n, int top, int C, const int* idx,
                     int E, const void* h, long long h_stride, int dt, cudaStream_t st) {
  if (n == 0) return 0;
  if (idx && !h) return -2;
  HYB_DISPATCH(dt, (combine_rows_kernel<bf16><<<n, 256, 0, st>>>((const bf16*)y, where, wt, (bf16*)out, top, C, idx, E, (const bf16*)h, h_stride)),
               (combine_rows_kernel<float><<<n, 256, 0, st>>>((const float*)y, where, wt, (float*)out, top, C, idx, E, (const float*)h, h_stride)));
  return (int)cudaGetLastError();
}

int hyb_act_mul_rows(const void* in, long long in_stride, void* out, long long rows, int F, int act, float limit, int dt,
                     cudaStream_t st) {
  long long total = rows * F;
  if (total == 0) return 0;
  if (act < 0 || act > 2) return -3;
  if (F % 8 == 0 && in_stride % 8 == 0 && (uintptr_t)in % 32 == 0 && (uintptr_t)out % 32 == 0) {
    long long total8 = total / 8;
    unsigned vb = (unsigned)((total8 + 255) / 256);
    HYB_DISPATCH(dt, (act_mul_rows_vec_kernel<bf16><<<vb, 256, 0, st>>>((const bf16*)in, in_stride, (bf16*)out, F, act, total8, limit)),
                 (act_mul_rows_vec_kernel<float><<<vb, 256, 0, st>>>((const float*)in, in_stride, (float*)out, F, act, total8, limit)));
    return (int)cudaGetLastError();
  }
  unsigned blocks = (unsigned)((total + 255) / 256);
  HYB_DISPATCH(dt, (act_mul_rows_kernel<bf16><<<blocks, 256, 0, st>>>((const bf16*)in, in_stride, (bf16*)out, F, act, total, limit)),
               (act_mul_rows_kernel<float><<<blocks, 256, 0, st>>>((const float*)in, in_stride, (float*)out, F, act, total, limit)));
  return (int)cudaGetLastError();
}

int hyb_scaled_branches(float* x, long long x_stride, const void* a, long long a_stride, const void* ls1, const void* b,
                        long long b_stride, const void* b2, long long b2_stride, const void* ls2, int rows, int C, int dt,
                        cudaStream_t st) {
  if (rows == 0) return 0;
  if (b2 && !b) return -2;
  HYB_DISPATCH(dt,
               (scaled_branches_kernel<bf16><<<rows, 256, 0, st>>>(x, x_stride, (const bf16*)a, a_stride, (const bf16*)ls1,
                                                                   (const bf16*)b, b_stride, (const bf16*)b2, b2_stride,
                                                                   (const bf16*)ls2, C)),
               (scaled_branches_kernel<float><<<rows, 256, 0, st>>>(x, x_stride, (const float*)a, a_stride,
                                                                    (const float*)ls1, (const float*)b, b_stride,
                                                                    (const float*)b2, b2_stride, (const float*)ls2, C)));
  return (int)cudaGetLastError();
}

}  // extern "C"

// =========================================================================================================
// post-norm blocks: norm over a whole projection before the rotation, the fixed-decay linear recurrence
// ("lightning" attention) in a token-scan and a chunked form, and the norm of a gated sum of two branches
// =========================================================================================================
namespace hyb {

// One block per token.  The query row (all H heads, H * D values) is divided by ITS root mean square over all H * D
// values (eps inside the root) and multiplied by qw [H * D]; then the first `nrot` entries of every head are rotated
// (entry 2i with 2i+1, angle pos * inv_freq[i]) and the row is stored in place.  The key row (G * D values, kw) gets
// the same treatment on its way into the slot's cache row, the values are copied behind it.  k == nullptr: a layer
// that borrows another layer's keys and values prepares its queries only.  Norm and rotation are fp32; a value is
// rounded once, after the rotation.  A thread owns both members of a rotated pair, so in-place stores race with no load.
template <typename T>
__global__ void full_norm_append_kernel(T* __restrict__ q, long long q_stride, const T* __restrict__ k, long long k_stride,
                                        const T* __restrict__ v, long long v_stride, const float* __restrict__ inv_freq,
                                        T* __restrict__ cache, long long slot_stride, const int* __restrict__ meta,
                                        const int* __restrict__ tok_seq, int H, int G, int D, int V, int nrot, float eps,
                                        const T* __restrict__ qw, const T* __restrict__ kw) {
  __shared__ float red[33];
  int t = blockIdx.x;
  const int* m = meta + 4 * tok_seq[t];
  int pos = m[3] + (t - m[0]);
  float fpos = (float)pos;
  for (int part = 0; part < (k ? 2 : 1); ++part) {
    const T* src = part == 0 ? q + (size_t)t * q_stride : k + (size_t)t * k_stride;
    T* dst = part == 0 ? q + (size_t)t * q_stride
                       : cache + (size_t)m[2] * slot_stride + (size_t)pos * (G * (D + V));
    const T* w = part == 0 ? qw : kw;
    int n = (part == 0 ? H : G) * D;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      float x = to_f(src[i]);
      ss += x * x;
    }
    float inv = 1.f / sqrtf(block_sum(ss, red) / n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      int d = i % D;
      if (d < nrot) {
        if (d & 1) continue;  // written by the owner of the even member
        float a = to_f(src[i]) * inv * to_f(w[i]), b = to_f(src[i + 1]) * inv * to_f(w[i + 1]), sn, cs;
        sincosf(fpos * inv_freq[d >> 1], &sn, &cs);
        dst[i] = from_f<T>(a * cs - b * sn);
        dst[i + 1] = from_f<T>(b * cs + a * sn);
      } else {
        dst[i] = from_f<T>(to_f(src[i]) * inv * to_f(w[i]));
      }
    }
  }
  if (k) {
    const T* vs = v + (size_t)t * v_stride;
    T* vd = cache + (size_t)m[2] * slot_stride + (size_t)pos * (G * (D + V)) + (size_t)G * D;
    for (int i = threadIdx.x; i < G * V; i += blockDim.x) vd[i] = vs[i];
  }
}

// Fixed-decay linear recurrence, token by token: S <- lam_h S + k v^T, o = S^T q, per head, S [D, V] fp32 in the slot.
// Grid (sequence, head, 32-column tile of V); thread (lane, dg) keeps S[dg + 8 i][v0 + lane] in registers (D <= 256),
// the eight row groups' partial read-outs meet in shared memory.  The form for one-token steps and short portions;
// o is written raw (fp32 [N, H * V]): the norm over all heads and the gate follow in norm_gate_rows_kernel.
// act != 0: q, k and v are pre-activations and their SiLU is taken (in fp32) where they are loaded.
#define LS_MAXI 32
__device__ __forceinline__ float lin_act(float x, int act) { return act ? siluf_(x) : x; }
template <typename T>
__global__ void __launch_bounds__(256) lightning_scan_kernel(const T* __restrict__ q, long long q_stride,
                                                             const T* __restrict__ k, long long k_stride,
                                                             const T* __restrict__ v, long long v_stride,
                                                             const float* __restrict__ decay, float* __restrict__ state,
                                                             const int* __restrict__ meta, float* __restrict__ oraw,
                                                             int H, int D, int V, int act) {
  __shared__ float qs[256], ks[256], part[8][33];
  const int* m = meta + 4 * blockIdx.x;
  int r0 = m[0], n = m[1], slot = m[2];
  int h = blockIdx.y, v0 = blockIdx.z * 32;
  int lane = threadIdx.x & 31, dg = threadIdx.x >> 5;
  int vc = v0 + lane;
  bool live = vc < V;
  float lam = decay[h];
  float* sp = state + (((size_t)slot * H + h) * D) * V;
  float S[LS_MAXI];
#pragma unroll
  for (int i = 0; i < LS_MAXI; ++i) {
    int d = dg + 8 * i;
    S[i] = d < D && live ? sp[(size_t)d * V + vc] : 0.f;
  }
  for (int t = r0; t < r0 + n; ++t) {
    for (int d = threadIdx.x; d < D; d += 256) {
      qs[d] = lin_act(to_f(q[(size_t)t * q_stride + (size_t)h * D + d]), act);
      ks[d] = lin_act(to_f(k[(size_t)t * k_stride + (size_t)h * D + d]), act);
    }
    float vv = live ? lin_act(to_f(v[(size_t)t * v_stride + (size_t)h * V + vc]), act) : 0.f;
    __syncthreads();
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < LS_MAXI; ++i) {
      int d = dg + 8 * i;
      if (d < D) {
        S[i] = lam * S[i] + ks[d] * vv;
        o += S[i] * qs[d];
      }
    }
    part[dg][lane] = o;
    __syncthreads();
    if (dg == 0 && live) {
      float a = 0.f;
#pragma unroll
      for (int g = 0; g < 8; ++g) a += part[g][lane];
      oraw[(size_t)t * H * V + (size_t)h * V + vc] = a;
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < LS_MAXI; ++i) {
      int d = dg + 8 * i;
      if (d < D) sp[(size_t)d * V + vc] = S[i];
    }
  }
}

// The same recurrence over prompt portions in chunks of LC_L = 64 tokens, parallel over the chunks.  With S the state
// before a chunk and positions t, s counted inside it,
//   o_t = lam^(t+1) S^T q_t + sum_{s <= t} lam^(t-s) (q_t . k_s) v_s          S' = lam^len S + sum_s lam^(len-1-s) k_s v_s^T
// so a chunk is four small matrix products instead of 64 dependent steps, and only S' = lam^len S + U chains the chunks
// of a sequence.  Powers of lam only have non-negative exponents, so nothing overflows however small lam is.  Three
// kernels over a chunk table ctab[c] = {first token row, tokens, sequence, 0} (chunks of a sequence in order) and
// stab[seq] = {first chunk, chunks}:
//   lightning_chunk_state_kernel  grid (chunk, head): U_c = sum_s lam^(len-1-s) k_s v_s^T -> scratch
//   lightning_chunk_scan_kernel   grid (sequence, head, slices of D*V): walks the sequence's chunks, replaces U_c by the
//                                 state BEFORE chunk c and leaves the final state in the slot
//   lightning_chunk_out_kernel    grid (chunk, head): decayed causal scores, weighted values, read-out of the state
//                                 before the chunk
// Everything is fp32 in shared memory: Q and K of the chunk transposed ([D][68]), the scores transposed ([s][t]), and per
// 32-column tile of V the value tile and the state tile [D][32].  A block loads Q and K and computes the scores once and
// walks the column tiles.  vec != 0 (rows 16-byte aligned, D a multiple of 8): a lane owns a token and fetches 8
// channels per load, so the transposed stores hit 32 different banks.  scratch is [chunks, H, D, V] fp32.
#define LC_L 64
#define LC_LP 68
#define LC_VT 32
// dst[d][t] = act(src[row0 + t, h * D + d]) for t < len, zero for the rest of the chunk (dst is [D][LC_LP]).
template <typename T>
__device__ __forceinline__ void load_chunk_transposed(float* __restrict__ dst, const T* __restrict__ src, long long stride,
                                                      int row0, int len, int h, int D, int act, int vec) {
  if (vec) {
    int d8n = D >> 3;
    for (int i = threadIdx.x; i < LC_L * d8n; i += 256) {
      int t = i & (LC_L - 1), d8 = i >> 6;  // a warp: 32 tokens of one group of 8 channels
      float f[8];
      if (t < len) {
        load8(src + (size_t)(row0 + t) * stride + (size_t)h * D + d8 * 8, f);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = 0.f;
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) dst[(d8 * 8 + e) * LC_LP + t] = t < len ? lin_act(f[e], act) : 0.f;
    }
    return;
  }
  for (int i = threadIdx.x; i < LC_L * D; i += 256) {
    int t = i / D, d = i - t * D;
    dst[d * LC_LP + t] = t < len ? lin_act(to_f(src[(size_t)(row0 + t) * stride + (size_t)h * D + d]), act) : 0.f;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) lightning_chunk_state_kernel(const T* __restrict__ k, long long k_stride,
                                                                    const T* __restrict__ v, long long v_stride,
                                                                    const float* __restrict__ decay,
                                                                    const int* __restrict__ ctab, float* __restrict__ scratch,
                                                                    int H, int D, int V, int act, int vec) {
  extern __shared__ __align__(16) float lsm[];
  float* Kt = lsm;                       // [D][LC_LP]
  float* Vs = Kt + (size_t)D * LC_LP;    // [LC_L][LC_VT], already times lam^(len-1-s)
  float* pw = Vs + LC_L * LC_VT;         // [LC_L + 1]
  const int* c = ctab + 4 * blockIdx.x;
  int row0 = c[0], len = c[1];
  int h = blockIdx.y;
  int tid = threadIdx.x, lane = tid & 31, tg = tid >> 5;
  for (int i = tid; i <= LC_L; i += 256) pw[i] = (float)pow((double)decay[h], (double)i);
  load_chunk_transposed(Kt, k, k_stride, row0, len, h, D, act, vec);
  float* up = scratch + (((size_t)blockIdx.x * H + h) * D) * V;
  for (int v0 = 0; v0 < V; v0 += LC_VT) {
    __syncthreads();  // pw and Kt are written; the previous tile is done with Vs
    for (int i = tid; i < LC_L * LC_VT; i += 256) {
      int t = i >> 5, cc = i & 31;
      Vs[i] = t < len && v0 + cc < V ? lin_act(to_f(v[(size_t)(row0 + t) * v_stride + (size_t)h * V + v0 + cc]), act) * pw[len - 1 - t] : 0.f;
    }
    __syncthreads();
    // thread (lane, tg) owns column lane of rows d = tg + 8 i, four rows at a time
    for (int i0 = 0; tg + 8 * i0 < D; i0 += 4) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      int dd[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) dd[u] = min(tg + 8 * (i0 + u), D - 1);  // rows past D: computed, not stored
      for (int s0 = 0; s0 < len; s0 += 4) {  // rows of Kt and Vs are zero past len
        float w0 = Vs[s0 * LC_VT + lane], w1 = Vs[(s0 + 1) * LC_VT + lane], w2 = Vs[(s0 + 2) * LC_VT + lane],
              w3 = Vs[(s0 + 3) * LC_VT + lane];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          float4 kv = *reinterpret_cast<const float4*>(Kt + dd[u] * LC_LP + s0);
          acc[u] += kv.x * w0 + kv.y * w1 + kv.z * w2 + kv.w * w3;
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        int d = tg + 8 * (i0 + u);
        if (d < D && v0 + lane < V) up[(size_t)d * V + v0 + lane] = acc[u];
      }
    }
  }
}

__global__ void lightning_chunk_scan_kernel(const float* __restrict__ decay, float* __restrict__ state,
                                            const int* __restrict__ meta, const int* __restrict__ ctab,
                                            const int* __restrict__ stab, float* __restrict__ scratch, int H, int D, int V) {
  // One thread per element of the [D, V] state.  Only the multiply-add chains the chunks: the U of eight chunks are
  // loaded together (independent loads in flight), then folded in order while the states before them are stored.
  __shared__ float s_full, s_last;
  int seq = blockIdx.x, h = blockIdx.y;
  int slot = meta[4 * seq + 2], c0 = stab[2 * seq], nc = stab[2 * seq + 1];
  if (threadIdx.x == 0) {
    double lam = (double)decay[h];
    s_full = (float)pow(lam, (double)LC_L);
    s_last = (float)pow(lam, (double)ctab[4 * (c0 + nc - 1) + 1]);  // only a sequence's last chunk can be short
  }
  __syncthreads();
  int e = blockIdx.z * blockDim.x + threadIdx.x;
  if (e >= D * V) return;
  const float full = s_full, last = s_last;
  const size_t cs = (size_t)H * D * V;  // floats between the same element of consecutive chunks
  float* sp = state + (((size_t)slot * H + h) * D) * V + e;
  float* u = scratch + (((size_t)c0 * H + h) * D) * V + e;
  float S = *sp;
  for (int c = 0; c < nc; c += 8) {
    float U[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) U[i] = c + i < nc ? u[(size_t)(c + i) * cs] : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (c + i < nc) {
        u[(size_t)(c + i) * cs] = S;  // the state before chunk c + i
        S = (c + i == nc - 1 ? last : full) * S + U[i];
      }
    }
  }
  *sp = S;
}

template <typename T>
__global__ void __launch_bounds__(256) lightning_chunk_out_kernel(const T* __restrict__ q, long long q_stride,
                                                                  const T* __restrict__ k, long long k_stride,
                                                                  const T* __restrict__ v, long long v_stride,
                                                                  const float* __restrict__ decay,
                                                                  const int* __restrict__ ctab,
                                                                  const float* __restrict__ scratch, float* __restrict__ oraw,
                                                                  int H, int D, int V, int act, int vec) {
  extern __shared__ __align__(16) float lsm[];
  float* Qt = lsm;                       // [D][LC_LP]
  float* Kt = Qt + (size_t)D * LC_LP;    // [D][LC_LP]
  float* At = Kt + (size_t)D * LC_LP;    // [LC_L][LC_LP]: At[s][t] = lam^(t-s) q_t . k_s for s <= t, else 0
  float* Vs = At + LC_L * LC_LP;         // [LC_L][LC_VT]
  float* Ss = Vs + LC_L * LC_VT;         // [D][LC_VT]: the state before the chunk
  float* pw = Ss + (size_t)D * LC_VT;    // [LC_L + 1]: lam^i
  const int* c = ctab + 4 * blockIdx.x;
  int row0 = c[0], len = c[1];
  int h = blockIdx.y;
  int tid = threadIdx.x, lane = tid & 31, tg = tid >> 5;
  const float* sp = scratch + (((size_t)blockIdx.x * H + h) * D) * V;
  for (int i = tid; i <= LC_L; i += 256) pw[i] = (float)pow((double)decay[h], (double)i);
  load_chunk_transposed(Qt, q, q_stride, row0, len, h, D, act, vec);
  load_chunk_transposed(Kt, k, k_stride, row0, len, h, D, act, vec);
  __syncthreads();
  int ty = tid >> 4, tx = tid & 15;
  {  // scores: thread (ty, tx) owns t = 4 ty .. 4 ty + 3 against s = 4 tx .. 4 tx + 3
    float a[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) a[i][j] = 0.f;
    if (tx <= ty) {  // blocks above the diagonal hold no visible pair
      for (int d = 0; d < D; ++d) {
        float4 qv = *reinterpret_cast<const float4*>(Qt + d * LC_LP + 4 * ty);
        float4 kv = *reinterpret_cast<const float4*>(Kt + d * LC_LP + 4 * tx);
        const float qa[4] = {qv.x, qv.y, qv.z, qv.w}, ka[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) a[i][j] += qa[i] * ka[j];
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int s_ = 4 * tx + j;
      float o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        int t = 4 * ty + i;
        o[i] = s_ <= t ? a[i][j] * pw[t - s_] : 0.f;
      }
      *reinterpret_cast<float4*>(At + s_ * LC_LP + 4 * ty) = make_float4(o[0], o[1], o[2], o[3]);
    }
  }
  __syncthreads();
  for (int v0 = 0; v0 < V; v0 += LC_VT) {
    int vc = v0 + lane;
    bool live = vc < V;
    for (int i = tid; i < D * LC_VT; i += 256) {
      int d = i >> 5, cc = i & 31;
      Ss[i] = v0 + cc < V ? sp[(size_t)d * V + v0 + cc] : 0.f;
    }
    for (int i = tid; i < LC_L * LC_VT; i += 256) {
      int t = i >> 5, cc = i & 31;
      Vs[i] = t < len && v0 + cc < V ? lin_act(to_f(v[(size_t)(row0 + t) * v_stride + (size_t)h * V + v0 + cc]), act) : 0.f;
    }
    __syncthreads();
    // outputs: thread (lane, tg) owns column v0 + lane of rows t = 8 tg .. 8 tg + 7
    float in[8], st[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) in[i] = st[i] = 0.f;
    int smax = min(len, 8 * tg + 8);
    for (int s_ = 0; s_ < smax; ++s_) {
      float vv = Vs[s_ * LC_VT + lane];
      float4 a0 = *reinterpret_cast<const float4*>(At + s_ * LC_LP + 8 * tg);
      float4 a1 = *reinterpret_cast<const float4*>(At + s_ * LC_LP + 8 * tg + 4);
      in[0] += a0.x * vv; in[1] += a0.y * vv; in[2] += a0.z * vv; in[3] += a0.w * vv;
      in[4] += a1.x * vv; in[5] += a1.y * vv; in[6] += a1.z * vv; in[7] += a1.w * vv;
    }
    for (int d = 0; d < D; ++d) {
      float sv = Ss[d * LC_VT + lane];
      float4 q0 = *reinterpret_cast<const float4*>(Qt + d * LC_LP + 8 * tg);
      float4 q1 = *reinterpret_cast<const float4*>(Qt + d * LC_LP + 8 * tg + 4);
      st[0] += q0.x * sv; st[1] += q0.y * sv; st[2] += q0.z * sv; st[3] += q0.w * sv;
      st[4] += q1.x * sv; st[5] += q1.y * sv; st[6] += q1.z * sv; st[7] += q1.w * sv;
    }
    if (live) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        int t = 8 * tg + i;
        if (t < len) oraw[(size_t)(row0 + t) * H * V + (size_t)h * V + vc] = in[i] + pw[t + 1] * st[i];
      }
    }
    __syncthreads();  // the next tile overwrites Vs and Ss
  }
}

// out[r, c] = o[r, c] / sqrt(mean_c(o[r, :]^2) + eps) * w[c] * sigmoid(g[r, c]): the RMS norm over ALL heads'
// concatenated read-outs (fp32 in) with its weight and the output gate, rounded once to the activation type.
template <typename T>
__global__ void norm_gate_rows_kernel(const float* __restrict__ o, const T* __restrict__ w, const T* __restrict__ g,
                                      long long g_stride, T* __restrict__ out, int n, float eps) {
  __shared__ float red[33];
  size_t r = blockIdx.x;
  const float* src = o + r * n;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) ss += src[i] * src[i];
  float inv = 1.f / sqrtf(block_sum(ss, red) / n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x)
    out[r * n + i] = from_f<T>(src[i] * inv * to_f(w[i]) * sigmoidf_(to_f(g[r * g_stride + i])));
}

// resid[r] += norm(a[r] + sigmoid(sg[r]) * b[r]) * w: the post-norm of a feed-forward whose always-on branch b is
// weighed by one sigmoid gate per token, and the residual sum, in one pass (fp32 arithmetic; b and sg optional).
// copy (optional, dense): the updated residual rounded to the activation type, for the next sublayer to read.
// kind 0: layer norm without bias, 1: RMS norm.
template <typename T>
__global__ void gated_sum_norm_kernel(const T* __restrict__ a, long long a_stride, const T* __restrict__ b,
                                      long long b_stride, const T* __restrict__ sg, long long sg_stride,
                                      const T* __restrict__ w, float* __restrict__ resid, long long r_stride, int n,
                                      float eps, int kind, T* __restrict__ copy) {
  __shared__ float red[33];
  size_t r = blockIdx.x;
  float gt = b ? (sg ? sigmoidf_(to_f(sg[r * sg_stride])) : 1.f) : 0.f;
  float mean = 0.f;
  if (kind == 0) {
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) s += to_f(a[r * a_stride + i]) + (b ? gt * to_f(b[r * b_stride + i]) : 0.f);
    mean = block_sum(s, red) / n;
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float y = to_f(a[r * a_stride + i]) + (b ? gt * to_f(b[r * b_stride + i]) : 0.f) - mean;
    ss += y * y;
  }
  float inv = 1.f / sqrtf(block_sum(ss, red) / n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float y = to_f(a[r * a_stride + i]) + (b ? gt * to_f(b[r * b_stride + i]) : 0.f) - mean;
    float x = resid[r * r_stride + i] + y * inv * to_f(w[i]);
    resid[r * r_stride + i] = x;
    if (copy) copy[r * n + i] = from_f<T>(x);
  }
}

}  // namespace hyb

extern "C" {

int hyb_full_norm_append(void* q, long long q_stride, const void* k, long long k_stride, const void* v, long long v_stride,
                         const float* inv_freq, void* cache, long long slot_stride, const int* meta, const int* tok_seq,
                         int N, int H, int G, int D, int V, int nrot, float eps, const void* qw, const void* kw, int dt,
                         cudaStream_t st) {
  if (N == 0) return 0;
  if (nrot > D || (nrot & 1) || (nrot > 0 && !inv_freq) || !qw || (k && (!kw || !v || !cache))) return -2;
  HYB_DISPATCH(dt,
               (full_norm_append_kernel<bf16><<<N, 256, 0, st>>>((bf16*)q, q_stride, (const bf16*)k, k_stride, (const bf16*)v,
                                                                 v_stride, inv_freq, (bf16*)cache, slot_stride, meta, tok_seq,
                                                                 H, G, D, V, nrot, eps, (const bf16*)qw, (const bf16*)kw)),
               (full_norm_append_kernel<float><<<N, 256, 0, st>>>((float*)q, q_stride, (const float*)k, k_stride,
                                                                  (const float*)v, v_stride, inv_freq, (float*)cache,
                                                                  slot_stride, meta, tok_seq, H, G, D, V, nrot, eps,
                                                                  (const float*)qw, (const float*)kw)));
  return (int)cudaGetLastError();
}

// variant 1: token scan; 2: chunks of 64 tokens (ctab [nchunks, 4], stab [nseq, 2] int32 and scratch
// [nchunks, H, D, V] fp32 on the device, see the kernels).  decay [H] fp32 on the device; oraw [N, H * V] fp32.
// act != 0: q, k, v are pre-activations; their SiLU is taken on load.
int hyb_lightning(const void* q, long long q_stride, const void* k, long long k_stride, const void* v, long long v_stride,
                  const float* decay, float* state, const int* meta, float* oraw, int nseq, int H, int D, int V,
                  int variant, int act, const int* ctab, const int* stab, int nchunks, float* scratch, int dt,
                  cudaStream_t st) {
  if (nseq == 0) return 0;
  if (D < 1 || D > 8 * LS_MAXI || V < 1) return -3;
  dim3 grid(nseq, H, (V + 31) / 32);
  if (variant == 1) {
    HYB_DISPATCH(dt,
                 (lightning_scan_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)q, q_stride, (const bf16*)k, k_stride,
                                                                    (const bf16*)v, v_stride, decay, state, meta, oraw, H, D, V, act)),
                 (lightning_scan_kernel<float><<<grid, 256, 0, st>>>((const float*)q, q_stride, (const float*)k, k_stride,
                                                                     (const float*)v, v_stride, decay, state, meta, oraw, H, D, V, act)));
    return (int)cudaGetLastError();
  }
  if (variant != 2) return -3;
  if (!ctab || !stab || !scratch || nchunks < 1) return -2;
  size_t sm1 = ((size_t)D * LC_LP + (size_t)LC_L * LC_VT + LC_L + 1 + 3) * sizeof(float);
  size_t sm3 = ((size_t)2 * D * LC_LP + (size_t)LC_L * LC_LP + (size_t)LC_L * LC_VT + (size_t)D * LC_VT + LC_L + 1 + 3) * sizeof(float);
  if (sm3 > 220 * 1024) return -3;
  dim3 cgrid(nchunks, H), sgrid(nseq, H, (D * V + 255) / 256);
  // 16-byte loads of q and k rows: every head's slice of every row starts on a 16-byte boundary
  int vec = D % 8 == 0 && q_stride % 8 == 0 && k_stride % 8 == 0 && (uintptr_t)q % 16 == 0 && (uintptr_t)k % 16 == 0;
  cudaError_t e;
  if (dt == 0) {
    if ((e = cudaFuncSetAttribute(lightning_chunk_state_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm1)) != cudaSuccess) return (int)e;
    if ((e = cudaFuncSetAttribute(lightning_chunk_out_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm3)) != cudaSuccess) return (int)e;
    lightning_chunk_state_kernel<bf16><<<cgrid, 256, sm1, st>>>((const bf16*)k, k_stride, (const bf16*)v, v_stride, decay, ctab,
                                                                scratch, H, D, V, act, vec);
    lightning_chunk_scan_kernel<<<sgrid, 256, 0, st>>>(decay, state, meta, ctab, stab, scratch, H, D, V);
    lightning_chunk_out_kernel<bf16><<<cgrid, 256, sm3, st>>>((const bf16*)q, q_stride, (const bf16*)k, k_stride, (const bf16*)v,
                                                              v_stride, decay, ctab, scratch, oraw, H, D, V, act, vec);
  } else {
    if ((e = cudaFuncSetAttribute(lightning_chunk_state_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm1)) != cudaSuccess) return (int)e;
    if ((e = cudaFuncSetAttribute(lightning_chunk_out_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm3)) != cudaSuccess) return (int)e;
    lightning_chunk_state_kernel<float><<<cgrid, 256, sm1, st>>>((const float*)k, k_stride, (const float*)v, v_stride, decay,
                                                                 ctab, scratch, H, D, V, act, vec);
    lightning_chunk_scan_kernel<<<sgrid, 256, 0, st>>>(decay, state, meta, ctab, stab, scratch, H, D, V);
    lightning_chunk_out_kernel<float><<<cgrid, 256, sm3, st>>>((const float*)q, q_stride, (const float*)k, k_stride,
                                                               (const float*)v, v_stride, decay, ctab, scratch, oraw, H, D, V, act, vec);
  }
  return (int)cudaGetLastError();
}

int hyb_norm_gate_rows(const float* o, const void* w, const void* g, long long g_stride, void* out, int rows, int n,
                       float eps, int dt, cudaStream_t st) {
  if (rows == 0) return 0;
  HYB_DISPATCH(dt, (norm_gate_rows_kernel<bf16><<<rows, 256, 0, st>>>(o, (const bf16*)w, (const bf16*)g, g_stride, (bf16*)out, n, eps)),
               (norm_gate_rows_kernel<float><<<rows, 256, 0, st>>>(o, (const float*)w, (const float*)g, g_stride, (float*)out, n, eps)));
  return (int)cudaGetLastError();
}

int hyb_gated_sum_norm(const void* a, long long a_stride, const void* b, long long b_stride, const void* sg,
                       long long sg_stride, const void* w, float* resid, long long r_stride, int rows, int n, float eps,
                       int kind, void* copy, int dt, cudaStream_t st) {
  if (rows == 0) return 0;
  if (kind < 0 || kind > 1 || !w) return -3;
  HYB_DISPATCH(dt,
               (gated_sum_norm_kernel<bf16><<<rows, 256, 0, st>>>((const bf16*)a, a_stride, (const bf16*)b, b_stride,
                                                                  (const bf16*)sg, sg_stride, (const bf16*)w, resid, r_stride,
                                                                  n, eps, kind, (bf16*)copy)),
               (gated_sum_norm_kernel<float><<<rows, 256, 0, st>>>((const float*)a, a_stride, (const float*)b, b_stride,
                                                                   (const float*)sg, sg_stride, (const float*)w, resid,
                                                                   r_stride, n, eps, kind, (float*)copy)));
  return (int)cudaGetLastError();
}

}  // extern "C"
