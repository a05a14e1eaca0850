// Sequence-mixer kernels for ragged batches with per-sequence state: zero-centred RMS norms on an fp32 residual stream,
// short causal convolutions with carried tails, the gated delta rule (one decay per head or per key channel) with its
// fp32 state, and sliding-window attention over cached low-rank latents (expanded keys/values for prompts, the
// absorbed form for single-token steps).
//
// Conventions.  A step carries B sequences; sequence b brings n_b = seq_off[b+1]-seq_off[b] new tokens that sit
// packed (no padding) at rows seq_off[b]..seq_off[b+1]-1 of every activation matrix, has past[b] tokens already
// folded into the state that lives in slot slots[b], and starts from an all-zero state when past[b] == 0 (the slot's
// old contents are then never read, so a slot can be reused without clearing it).  Activations are `T` (float or
// bf16, `dtype` 0 / 1); everything that enters a norm, a softmax or a recurrence is converted to fp32 first and the
// arithmetic is fp32.  This file is built WITHOUT fast-math: the fp32 mode is meant to be exact to rounding.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
  return v;
}
// sum over the block (blockDim.x a multiple of 32, at most 1024); every thread gets the result
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[w] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += red[i];
  return t;
}
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// ------------------------------------------------------------------------------------------------------------------
// RMS norm: y = x / sqrt(mean(x^2) + eps) * (offset + w).  One block per row.  Optional gather of the row through
// `ids` (token embedding + norm in one pass).
// ------------------------------------------------------------------------------------------------------------------
template <typename Tin, typename Tw, typename Tout>
__global__ void rmsnorm_kernel(const Tin* __restrict__ x, long ldx, const int64_t* __restrict__ ids, const Tw* __restrict__ w,
                               float offset, float eps, Tout* __restrict__ y, long ldy, int n) {
  __shared__ float red[32];
  const long row = blockIdx.x;
  const Tin* xr = x + (ids ? (long)ids[row] : row) * ldx;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) { float v = ldf(xr + i); ss += v * v; }
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x) stf(y + row * ldy + i, ldf(xr + i) * r * (offset + ldf(w + i)));
}

// out[row, 0:n] = act(in[row, 0:n]) on column slices; act 0: copy, 1: relu(x)^2, 2: silu, 3: gelu_tanh
template <typename Tin, typename Tout>
__global__ void slice_act_kernel(const Tin* __restrict__ in, long ldi, Tout* __restrict__ out, long ldo, long rows, int n, int act) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * n) return;
  const long r = idx / n; const int c = (int)(idx - r * n);
  float v = ldf(in + r * ldi + c);
  if (act == 1) { v = fmaxf(v, 0.f); v = v * v; }
  else if (act == 2) v = v * sigmoidf_(v);
  else if (act == 3) v = 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
  stf(out + r * ldo + c, v);
}

// the same on bf16 with 16-byte accesses: 8 columns per thread (n, both row strides and both base addresses multiples of 8 elements)
__global__ void slice_act_vec8_kernel(const __nv_bfloat16* __restrict__ in, long ldi, __nv_bfloat16* __restrict__ out, long ldo,
                                      long rows, int n8, int act) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * n8) return;
  const long r = idx / n8; const int c = (int)(idx - r * n8) * 8;
  uint4 raw = *reinterpret_cast<const uint4*>(in + r * ldi + c);
  __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 v = __bfloat1622float2(h2[i]);
    if (act == 1) { v.x = fmaxf(v.x, 0.f); v.x *= v.x; v.y = fmaxf(v.y, 0.f); v.y *= v.y; }
    else if (act == 2) { v.x = v.x * sigmoidf_(v.x); v.y = v.y * sigmoidf_(v.y); }
    else if (act == 3) {
      v.x = 0.5f * v.x * (1.f + tanhf(0.7978845608028654f * (v.x + 0.044715f * v.x * v.x * v.x)));
      v.y = 0.5f * v.y * (1.f + tanhf(0.7978845608028654f * (v.y + 0.044715f * v.y * v.y * v.y)));
    }
    h2[i] = __floats2bfloat162_rn(v.x, v.y);
  }
  *reinterpret_cast<uint4*>(out + r * ldo + c) = raw;
}

// ------------------------------------------------------------------------------------------------------------------
// Short causal convolution per channel + SiLU.  in: [tokens, ldi] (C channels from column 0), w: [C, taps] with the
// last tap on the current token, tail: [slots, taps-1, C] = the last taps-1 inputs of every sequence.
// ------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void short_conv_kernel(const T* __restrict__ in, long ldi, const T* __restrict__ w, const T* __restrict__ tail,
                                  const int* __restrict__ tok_seq, const int* __restrict__ seq_off, const int* __restrict__ slots,
                                  const int* __restrict__ past, T* __restrict__ out, long ldo, long tokens, int C, int taps) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= tokens * C) return;
  const long tok = idx / C; const int c = (int)(idx - tok * C);
  const int b = tok_seq[tok];
  const int t = (int)(tok - seq_off[b]);
  const bool has_past = past[b] > 0;
  const T* tl = tail + (long)slots[b] * (taps - 1) * C;
  float acc = 0.f;
  for (int k = 0; k < taps; ++k) {
    const int tp = t - k;
    float v;
    if (tp >= 0) v = ldf(in + (tok - k) * ldi + c);
    else v = has_past ? ldf(tl + (long)(taps - 1 + tp) * C + c) : 0.f;
    acc += ldf(w + (long)c * taps + (taps - 1 - k)) * v;
  }
  stf(out + tok * ldo + c, acc * sigmoidf_(acc));
}

// bf16 with 16-byte accesses: a thread owns 8 adjacent channels of one token (C, the row strides and the base addresses are
// multiples of 8 elements); the 8·TAPS weights of its channels are contiguous and come in as TAPS 16-byte loads
template <int TAPS>
__global__ void short_conv_vec8_kernel(const __nv_bfloat16* __restrict__ in, long ldi, const __nv_bfloat16* __restrict__ w,
                                       const __nv_bfloat16* __restrict__ tail, const int* __restrict__ tok_seq,
                                       const int* __restrict__ seq_off, const int* __restrict__ slots, const int* __restrict__ past,
                                       __nv_bfloat16* __restrict__ out, long ldo, long tokens, int C) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const int C8 = C >> 3;
  if (idx >= tokens * C8) return;
  const long tok = idx / C8; const int c = (int)(idx - tok * C8) * 8;
  const int b = tok_seq[tok];
  const int t = (int)(tok - seq_off[b]);
  const bool has_past = past[b] > 0;
  const __nv_bfloat16* tl = tail + (long)slots[b] * (TAPS - 1) * C;
  uint4 wraw[TAPS];
#pragma unroll
  for (int k = 0; k < TAPS; ++k) wraw[k] = reinterpret_cast<const uint4*>(w + (long)c * TAPS)[k];
  const __nv_bfloat16* wv = reinterpret_cast<const __nv_bfloat16*>(wraw);      // wv[i * TAPS + j]: channel c + i, tap j
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
  for (int k = 0; k < TAPS; ++k) {
    const int tp = t - k;
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if (tp >= 0) raw = *reinterpret_cast<const uint4*>(in + (tok - k) * ldi + c);
    else if (has_past) raw = *reinterpret_cast<const uint4*>(tl + (long)(TAPS - 1 + tp) * C + c);
    const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += __bfloat162float(wv[i * TAPS + (TAPS - 1 - k)]) * __bfloat162float(x[i]);
  }
  uint4 res;
  __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
  for (int i = 0; i < 4; ++i) r2[i] = __floats2bfloat162_rn(acc[2 * i] * sigmoidf_(acc[2 * i]), acc[2 * i + 1] * sigmoidf_(acc[2 * i + 1]));
  *reinterpret_cast<uint4*>(out + tok * ldo + c) = res;
}

template <typename T>
__global__ void conv_tail_kernel(const T* __restrict__ in, long ldi, T* __restrict__ tail, const int* __restrict__ seq_off,
                                 const int* __restrict__ slots, const int* __restrict__ past, int B, int C, int taps) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long)B * C) return;
  const int b = (int)(idx / C), c = (int)(idx - (long)b * C);
  const int n = seq_off[b + 1] - seq_off[b];
  const bool has_past = past[b] > 0;
  T* tl = tail + (long)slots[b] * (taps - 1) * C;
  for (int i = 0; i < taps - 1; ++i) {          // ascending: new[i] only reads old[i + n], never a rewritten entry
    const int tp = n - (taps - 1) + i;
    float v;
    if (tp >= 0) v = ldf(in + ((long)seq_off[b] + tp) * ldi + c);
    else v = (has_past && i + n < taps - 1) ? ldf(tl + (long)(i + n) * C + c) : 0.f;
    stf(tl + (long)i * C + c, v);
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Gated delta rule.  Per head, with S [D, V] in fp32:   S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;
// o = S^T q.  q and k arrive after the convolution, are normalised here to unit length per head (eps inside the
// root) and q is scaled by D^-1/2.  g = exp(-exp(A_log) softplus(a + dt_bias)) per head (chan == 0) or per key channel
// (chan == 1); beta = sigmoid(b).  Columns of S are independent: a block owns `VT` of them for one (sequence, head);
// every column is shared by R lanes (R a power of two, adjacent lanes of one warp) that each keep DPT consecutive rows
// of it in registers, so a token costs 3·DPT fused multiply-adds per lane and log2(R) shuffle rounds.  A first kernel
// prepares the per-token quantities (unit vectors, decays, write strengths) once; the scan stages them
// through shared memory `CT` at a time (rows of lane r at offset r·(DPT+4): 16-byte loads without bank conflicts), so
// the serial part only touches registers and shared memory.
// ------------------------------------------------------------------------------------------------------------------
constexpr int CT = 16;

// Per token: unit-length keys and queries (queries also times D^-1/2) per key head in fp32, their dot product, the write
// strength beta = sigmoid(b) and the decay g per head (or per head and key channel).  One warp per (token, key head);
// the value heads of a group share its work.
template <typename T>
__global__ void delta_prep_kernel(const T* __restrict__ qkv, long ldq, int koff, const T* __restrict__ a, long lda,
                                  const T* __restrict__ bl, long ldb, const T* __restrict__ A_log, const T* __restrict__ dt_bias,
                                  float* __restrict__ qn, float* __restrict__ kn, float* __restrict__ kq, float* __restrict__ g,
                                  float* __restrict__ beta, long tokens, int H, int KH, int D, int chan) {
  const long wid = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= tokens * KH) return;
  const long tok = wid / KH; const int kh = (int)(wid - tok * KH);
  const T* qr = qkv + tok * ldq + kh * D; const T* kr = qkv + tok * ldq + koff + kh * D;
  float qq = 0.f, kk = 0.f;
  for (int i = lane; i < D; i += 32) { const float x = ldf(qr + i), y = ldf(kr + i); qq += x * x; kk += y * y; }
  qq = warp_sum(qq); kk = warp_sum(kk);
  const float qsc = (1.f / sqrtf((float)D)) / sqrtf(qq + 1e-6f), ksc = 1.f / sqrtf(kk + 1e-6f);
  float dot = 0.f;
  for (int i = lane; i < D; i += 32) {
    const float x = ldf(qr + i) * qsc, y = ldf(kr + i) * ksc;
    qn[(tok * KH + kh) * D + i] = x; kn[(tok * KH + kh) * D + i] = y; dot += x * y;
  }
  dot = warp_sum(dot);
  if (lane == 0) kq[tok * KH + kh] = dot;
  const int group = H / KH;
  for (int hh = 0; hh < group; ++hh) {
    const int h = kh * group + hh;
    const float rate = expf(ldf(A_log + h));
    if (chan) {
      for (int i = lane; i < D; i += 32)
        g[(tok * H + h) * D + i] = expf(-rate * softplusf_(ldf(a + tok * lda + h * D + i) + ldf(dt_bias + h * D + i)));
    } else if (lane == 0) {
      g[tok * H + h] = expf(-rate * softplusf_(ldf(a + tok * lda + h) + ldf(dt_bias + h)));
    }
    if (lane == 0) beta[tok * H + h] = sigmoidf_(ldf(bl + tok * ldb + h));
  }
}

template <typename T, int DPT>
__global__ void __launch_bounds__(256, DPT <= 16 ? 2 : 1)   // two blocks per SM where 128 registers hold the rows
delta_scan_kernel(const T* __restrict__ qkv, long ldq, int voff, const float* __restrict__ qn, const float* __restrict__ kn,
                  const float* __restrict__ kqs, const float* __restrict__ gs, const float* __restrict__ betas,
                  float* __restrict__ S, const int* __restrict__ seq_off, const int* __restrict__ slots,
                  const int* __restrict__ past, float* __restrict__ out, int H, int KH, int D, int V, int R, int VT, int chan) {
  extern __shared__ __align__(16) float sm[];
  constexpr int PS = DPT + 4;                   // padded stride of one lane's rows
  const int b = blockIdx.x / H, h = blockIdx.x % H, kh = h / (H / KH);
  const int j0 = blockIdx.y * VT;
  const int Dr = R * DPT;                       // rows covered (rows >= D hold zeros)
  const int Dp = R * PS;                        // floats per staged token
  float* sk = sm;                               // [CT][Dp]
  float* sq = sk + CT * Dp;                     // [CT][Dp]
  float* sg = sq + CT * Dp;                     // [CT][Dp] (chan) or [CT]
  float* sv = sg + CT * (chan ? Dp : 4);        // [CT][VT]
  float* sbeta = sv + CT * VT;                  // [CT]
  float* skq = sbeta + CT;                      // [CT]
  const int tid = threadIdx.x, nth = blockDim.x;
  const int r = tid % R, jj = tid / R, j = j0 + jj;
  const bool col_ok = jj < VT && j < V;
  const int n = seq_off[b + 1] - seq_off[b];
  const long tok0 = seq_off[b];
  float* Sg = S + ((long)slots[b] * H + h) * (long)D * V;
  float s[DPT];
#pragma unroll
  for (int d = 0; d < DPT; ++d) {
    const int i = r * DPT + d;
    s[d] = (past[b] > 0 && col_ok && i < D) ? Sg[(long)i * V + j] : 0.f;
  }
  for (int c0 = 0; c0 < n; c0 += CT) {
    const int ct = min(CT, n - c0);
    __syncthreads();
    for (int e = tid; e < ct * Dr; e += nth) {
      const int t = e / Dr, i = e - t * Dr;
      const int pos = t * Dp + (i / DPT) * PS + (i % DPT);
      const long row = tok0 + c0 + t;
      const bool in = i < D;
      sk[pos] = in ? kn[(row * KH + kh) * D + i] : 0.f;
      sq[pos] = in ? qn[(row * KH + kh) * D + i] : 0.f;
      if (chan) sg[pos] = in ? gs[(row * H + h) * D + i] : 1.f;
    }
    for (int e = tid; e < ct * VT; e += nth) {
      const int t = e / VT, c = e - t * VT;
      sv[e] = (j0 + c < V) ? ldf(qkv + (tok0 + c0 + t) * ldq + voff + h * V + j0 + c) : 0.f;
    }
    for (int t = tid; t < ct; t += nth) {
      const long row = tok0 + c0 + t;
      sbeta[t] = betas[row * H + h];
      skq[t] = kqs[row * KH + kh];
      if (!chan) sg[t] = gs[row * H + h];
    }
    __syncthreads();
    // every thread walks the tokens (lanes of idle columns included: the shuffles below name the whole warp)
    for (int t = 0; t < ct; ++t) {
      float kr[DPT];
      float pk[4] = {0.f, 0.f, 0.f, 0.f}, pq[4] = {0.f, 0.f, 0.f, 0.f};
      const float4* k4 = reinterpret_cast<const float4*>(sk + t * Dp + r * PS);
      const float4* q4 = reinterpret_cast<const float4*>(sq + t * Dp + r * PS);
      const float4* g4 = reinterpret_cast<const float4*>(sg + t * Dp + r * PS);
      const float g0 = chan ? 1.f : sg[t];
#pragma unroll
      for (int d4 = 0; d4 < DPT / 4; ++d4) {
        const float4 kx = k4[d4], qx = q4[d4];
        float4 gx = make_float4(g0, g0, g0, g0);
        if (chan) gx = g4[d4];
        kr[4 * d4] = kx.x; kr[4 * d4 + 1] = kx.y; kr[4 * d4 + 2] = kx.z; kr[4 * d4 + 3] = kx.w;
        s[4 * d4] *= gx.x; s[4 * d4 + 1] *= gx.y; s[4 * d4 + 2] *= gx.z; s[4 * d4 + 3] *= gx.w;
        pk[0] += s[4 * d4] * kx.x; pk[1] += s[4 * d4 + 1] * kx.y; pk[2] += s[4 * d4 + 2] * kx.z; pk[3] += s[4 * d4 + 3] * kx.w;
        pq[0] += s[4 * d4] * qx.x; pq[1] += s[4 * d4 + 1] * qx.y; pq[2] += s[4 * d4 + 2] * qx.z; pq[3] += s[4 * d4 + 3] * qx.w;
      }
      float sk_ = (pk[0] + pk[1]) + (pk[2] + pk[3]), sq_ = (pq[0] + pq[1]) + (pq[2] + pq[3]);
      for (int m = R >> 1; m > 0; m >>= 1) { sk_ += __shfl_xor_sync(0xffffffffu, sk_, m); sq_ += __shfl_xor_sync(0xffffffffu, sq_, m); }
      const float u = sbeta[t] * ((jj < VT ? sv[t * VT + jj] : 0.f) - sk_);
#pragma unroll
      for (int d = 0; d < DPT; ++d) s[d] += kr[d] * u;
      if (r == 0 && col_ok) out[(tok0 + c0 + t) * (long)(H * V) + h * V + j] = sq_ + skq[t] * u;
    }
  }
  if (col_ok) {
#pragma unroll
    for (int d = 0; d < DPT; ++d) { const int i = r * DPT + d; if (i < D) Sg[(long)i * V + j] = s[d]; }
  }
}

// y[tok, h, :] = o / rms(o over V) * w * act(gate[tok, h, :]);  act 0: silu, 1: sigmoid.  One warp per (token, head).
template <typename T>
__global__ void gated_rmsnorm_kernel(const float* __restrict__ o, const T* __restrict__ gate, long ldg, const T* __restrict__ w,
                                     float eps, int act, T* __restrict__ y, long ldy, long rows, int H, int V) {
  const long wid = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= rows * H) return;
  const long tok = wid / H; const int h = (int)(wid - tok * H);
  const float* orow = o + (tok * H + h) * (long)V;
  float ss = 0.f;
  for (int i = lane; i < V; i += 32) ss += orow[i] * orow[i];
  ss = warp_sum(ss);
  const float rr = 1.f / sqrtf(ss / (float)V + eps);
  for (int i = lane; i < V; i += 32) {
    const float g = ldf(gate + tok * ldg + h * V + i);
    const float ga = act == 0 ? g * sigmoidf_(g) : sigmoidf_(g);
    stf(y + tok * ldy + h * V + i, orow[i] * rr * ldf(w + i) * ga);
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Latent cache: ring[slot][p % ring_len] holds the latent of position p; ring_len >= window.  `gather` lays out, for every
// sequence, the still-visible cached latents followed by the step's new ones (ext rows); `write` stores the new ones.
// ------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void latent_gather_kernel(const T* __restrict__ ring, const T* __restrict__ cnew, const int* __restrict__ ext_seq,
                                     const int* __restrict__ ext_off, const int* __restrict__ seq_off, const int* __restrict__ slots,
                                     const int* __restrict__ past, T* __restrict__ ext, long rows, int C, int ring_len) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * C) return;
  const long e = idx / C; const int c = (int)(idx - e * C);
  const int b = ext_seq[e];
  const int ie = (int)(e - ext_off[b]);
  const int n = seq_off[b + 1] - seq_off[b];
  const int npast = ext_off[b + 1] - ext_off[b] - n;
  if (ie < npast) {
    const int pos = past[b] - npast + ie;
    ext[idx] = ring[((long)slots[b] * ring_len + pos % ring_len) * C + c];
  } else {
    ext[idx] = cnew[((long)seq_off[b] + ie - npast) * C + c];
  }
}

template <typename T>
__global__ void latent_write_kernel(T* __restrict__ ring, const T* __restrict__ cnew, const int* __restrict__ tok_seq,
                                    const int* __restrict__ seq_off, const int* __restrict__ slots, const int* __restrict__ past,
                                    long tokens, int C, int ring_len) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= tokens * C) return;
  const long tok = idx / C; const int c = (int)(idx - tok * C);
  const int b = tok_seq[tok];
  const int t = (int)(tok - seq_off[b]), n = seq_off[b + 1] - seq_off[b];
  if (t < n - ring_len) return;                 // an older token of this step would be overwritten anyway
  const int pos = past[b] + t;
  ring[((long)slots[b] * ring_len + pos % ring_len) * C + c] = cnew[idx];
}

// ------------------------------------------------------------------------------------------------------------------
// Sliding-window attention on expanded keys / values.  q: [tokens, H*D]; kv: [ext rows, H*D + H*V] (keys, then values);
// query t of sequence b sits at ext row ext_off[b] + npast + t and sees the `window` ext rows ending at its own, never
// crossing the start of its sequence's ext range.  One warp per (token, head): lanes take keys for the scores and value
// channels for the output; softmax in fp32, streamed 32 keys at a time.  The head's output is multiplied by
// sigmoid(gate[tok, h]) when a gate is given.
// ------------------------------------------------------------------------------------------------------------------
constexpr int ATT_MAXV = 8;    // value channels per lane: V <= 256

template <typename T>
__global__ void window_attention_kernel(const T* __restrict__ q, long ldq, const T* __restrict__ kv, long ldkv, const T* __restrict__ gate,
                                        long ldg, const int* __restrict__ tok_seq, const int* __restrict__ seq_off,
                                        const int* __restrict__ ext_off, T* __restrict__ y, long ldy, long tokens, int H, int D,
                                        int V, int window, float scale) {
  extern __shared__ float sm[];
  const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long wid = (long)blockIdx.x * (blockDim.x >> 5) + wib;
  if (wid >= tokens * H) return;                 // no block-level sync below
  const long tok = wid / H; const int h = (int)(wid - tok * H);
  const int b = tok_seq[tok];
  const int n = seq_off[b + 1] - seq_off[b];
  const int npast = ext_off[b + 1] - ext_off[b] - n;
  const long eq = (long)ext_off[b] + npast + (tok - seq_off[b]);
  long e0 = eq - window + 1;
  if (e0 < ext_off[b]) e0 = ext_off[b];
  float* qs = sm + wib * D;
  for (int i = lane; i < D; i += 32) qs[i] = ldf(q + tok * ldq + h * D + i) * scale;
  __syncwarp();
  float m = -INFINITY, l = 0.f, acc[ATT_MAXV];
#pragma unroll
  for (int i = 0; i < ATT_MAXV; ++i) acc[i] = 0.f;
  for (long e = e0; e <= eq; e += 32) {
    const long mine = e + lane;
    float sc = -INFINITY;
    if (mine <= eq) {
      const T* kr = kv + mine * ldkv + h * D;
      float d = 0.f;
      for (int i = 0; i < D; ++i) d += qs[i] * ldf(kr + i);
      sc = d;
    }
    const float mn = fmaxf(m, warp_max(sc));
    const float corr = expf(m - mn);             // m = -inf on the first block: exp(-inf) = 0
    const float p = mine <= eq ? expf(sc - mn) : 0.f;
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < ATT_MAXV; ++i) acc[i] *= corr;
    const int cnt = (int)min((long)32, eq - e + 1);
    for (int k = 0; k < cnt; ++k) {
      const float pk = __shfl_sync(0xffffffffu, p, k);
      const T* vr = kv + (e + k) * ldkv + (long)H * D + h * V;
#pragma unroll
      for (int i = 0; i < ATT_MAXV; ++i) { const int c = lane + 32 * i; if (c < V) acc[i] += pk * ldf(vr + c); }
    }
    m = mn;
  }
  const float g = gate ? sigmoidf_(ldf(gate + tok * ldg + h)) : 1.f;
  const float inv = g / l;
#pragma unroll
  for (int i = 0; i < ATT_MAXV; ++i) { const int c = lane + 32 * i; if (c < V) stf(y + tok * ldy + h * V + c, acc[i] * inv); }
}

// ------------------------------------------------------------------------------------------------------------------
// The same attention on the tensor cores (bf16 operands, fp32 accumulation and softmax): a block of 4 warps owns 64
// consecutive queries of one (sequence, head) — 16 per warp, held as A fragments — and walks the key rows its queries can
// see in tiles of 64 staged through shared memory: S = Q Kᵀ with mma.m16n8k16, online softmax on the accumulator
// fragments, P re-packed as A fragments, O += P V with the V fragments fetched by ldmatrix.trans.  Query tiles are
// listed by the host (qt_seq / qt_start), so ragged batches cost no empty blocks.
// ------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int D, int V>
__global__ void __launch_bounds__(128)
window_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, long ldq, const __nv_bfloat16* __restrict__ kv, long ldkv,
                            const __nv_bfloat16* __restrict__ gate, long ldg, const int* __restrict__ qt_seq,
                            const int* __restrict__ qt_start, const int* __restrict__ seq_off, const int* __restrict__ ext_off,
                            __nv_bfloat16* __restrict__ y, long ldy, int H, int window, float scale) {
  constexpr int KT = 64, KS = D + 8, VS = V + 8;
  __shared__ __align__(16) __nv_bfloat16 Ks[KT * KS];
  __shared__ __align__(16) __nv_bfloat16 Vs[KT * VS];
  const int h = blockIdx.y, b = qt_seq[blockIdx.x], t0 = qt_start[blockIdx.x];
  const int n = seq_off[b + 1] - seq_off[b];
  const int elo = ext_off[b], ehi = ext_off[b + 1], npast = ehi - elo - n;
  const long tokbase = seq_off[b];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
  const int r0 = t0 + warp * 16 + gid, r1 = r0 + 8;                    // this lane's two query rows
  const int e0 = elo + npast + r0, e1 = e0 + 8;                          // their key rows
  uint32_t qf[D / 16][4];
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    const int col = h * D + kk * 16 + tig * 2;
    qf[kk][0] = r0 < n ? *reinterpret_cast<const uint32_t*>(q + (tokbase + r0) * ldq + col) : 0u;
    qf[kk][1] = r1 < n ? *reinterpret_cast<const uint32_t*>(q + (tokbase + r1) * ldq + col) : 0u;
    qf[kk][2] = r0 < n ? *reinterpret_cast<const uint32_t*>(q + (tokbase + r0) * ldq + col + 8) : 0u;
    qf[kk][3] = r1 < n ? *reinterpret_cast<const uint32_t*>(q + (tokbase + r1) * ldq + col + 8) : 0u;
  }
  float o[V / 8][4];
#pragma unroll
  for (int j = 0; j < V / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;              // l: this lane's share of the row sums
  const int eq_first = elo + npast + t0, eq_last = elo + npast + min(t0 + 63, n - 1);
  const int ew0 = eq_first + warp * 16;                                   // first key row of this warp's queries
  int kbeg = eq_first - window + 1;
  if (kbeg < elo) kbeg = elo;
  for (int k0 = kbeg; k0 <= eq_last; k0 += KT) {
    __syncthreads();
    for (int c = threadIdx.x; c < KT * (D / 8); c += 128) {
      const int row = c / (D / 8), ch = c - row * (D / 8);
      uint4 val = make_uint4(0u, 0u, 0u, 0u);
      if (k0 + row < ehi) val = *reinterpret_cast<const uint4*>(kv + (long)(k0 + row) * ldkv + h * D + ch * 8);
      *reinterpret_cast<uint4*>(&Ks[row * KS + ch * 8]) = val;
    }
    for (int c = threadIdx.x; c < KT * (V / 8); c += 128) {
      const int row = c / (V / 8), ch = c - row * (V / 8);
      uint4 val = make_uint4(0u, 0u, 0u, 0u);
      if (k0 + row < ehi) val = *reinterpret_cast<const uint4*>(kv + (long)(k0 + row) * ldkv + (long)H * D + h * V + ch * 8);
      *reinterpret_cast<uint4*>(&Vs[row * VS + ch * 8]) = val;
    }
    __syncthreads();
    if (k0 > ew0 + 15 || k0 + KT - 1 <= ew0 - window) continue;          // nothing in this tile for the warp's 16 queries
    float sacc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) { sacc[j][0] = sacc[j][1] = sacc[j][2] = sacc[j][3] = 0.f; }
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const __nv_bfloat16* kr = &Ks[(j * 8 + gid) * KS + kk * 16 + tig * 2];
        mma_bf16(sacc[j], qf[kk], *reinterpret_cast<const uint32_t*>(kr), *reinterpret_cast<const uint32_t*>(kr + 8));
      }
    }
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int key = k0 + j * 8 + tig * 2 + (c & 1), eq = c < 2 ? e0 : e1;
        const bool valid = key <= eq && key > eq - window;
        const float sv = valid ? sacc[j][c] * scale : -INFINITY;
        sacc[j][c] = sv;
        if (c < 2) mx0 = fmaxf(mx0, sv); else mx1 = fmaxf(mx1, sv);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float c0 = mn0 == -INFINITY ? 1.f : __expf(m0 - mn0), c1 = mn1 == -INFINITY ? 1.f : __expf(m1 - mn1);
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float sv = sacc[j][c];
        const float pv = sv == -INFINITY ? 0.f : __expf(sv - (c < 2 ? mn0 : mn1));
        sacc[j][c] = pv;
        if (c < 2) s0 += pv; else s1 += pv;
      }
    }
    l0 = l0 * c0 + s0; l1 = l1 * c1 + s1; m0 = mn0; m1 = mn1;
#pragma unroll
    for (int j = 0; j < V / 8; ++j) { o[j][0] *= c0; o[j][1] *= c0; o[j][2] *= c1; o[j][3] *= c1; }
#pragma unroll
    for (int k2 = 0; k2 < 4; ++k2) {
      uint32_t a[4];
      a[0] = pack_bf16(sacc[2 * k2][0], sacc[2 * k2][1]); a[1] = pack_bf16(sacc[2 * k2][2], sacc[2 * k2][3]);
      a[2] = pack_bf16(sacc[2 * k2 + 1][0], sacc[2 * k2 + 1][1]); a[3] = pack_bf16(sacc[2 * k2 + 1][2], sacc[2 * k2 + 1][3]);
      const uint32_t vrow = (uint32_t)__cvta_generic_to_shared(&Vs[(k2 * 16 + (lane & 15)) * VS]);
#pragma unroll
      for (int j = 0; j < V / 8; ++j) {
        uint32_t b0, b1;
        asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(b0), "=r"(b1) : "r"(vrow + j * 16));
        mma_bf16(o[j], a, b0, b1);
      }
    }
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float g0 = (gate && r0 < n) ? sigmoidf_(__bfloat162float(gate[(tokbase + r0) * ldg + h])) : 1.f;
  const float g1 = (gate && r1 < n) ? sigmoidf_(__bfloat162float(gate[(tokbase + r1) * ldg + h])) : 1.f;
  const float i0 = g0 / l0, i1 = g1 / l1;
#pragma unroll
  for (int j = 0; j < V / 8; ++j) {
    const int col = h * V + j * 8 + tig * 2;
    if (r0 < n) *reinterpret_cast<uint32_t*>(y + (tokbase + r0) * ldy + col) = pack_bf16(o[j][0] * i0, o[j][1] * i0);
    if (r1 < n) *reinterpret_cast<uint32_t*>(y + (tokbase + r1) * ldy + col) = pack_bf16(o[j][2] * i1, o[j][3] * i1);
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Single-token steps in the absorbed form: the query already carries the key up-projection (qa [B, H, C], fp32), so the
// scores and the weighted sum run on the cached latents themselves; the new token's latent (cnew [B, C]) is position
// past[b], the others come from the ring.  out: [B, H, C] fp32 = softmax-weighted latent per head (the value
// up-projection follows as a batched matrix product).  One warp per (sequence, head).
// ------------------------------------------------------------------------------------------------------------------
constexpr int ABS_MAXC = 32;   // latent channels per lane: C <= 1024

template <typename T>
__global__ void latent_decode_kernel(const float* __restrict__ qa, const T* __restrict__ ring, const T* __restrict__ cnew,
                                     const int* __restrict__ slots, const int* __restrict__ past, float* __restrict__ out, int B, int H,
                                     int C, int ring_len, int window, float scale) {
  extern __shared__ float sm[];
  const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long wid = (long)blockIdx.x * (blockDim.x >> 5) + wib;
  if (wid >= (long)B * H) return;
  const int b = (int)(wid / H), h = (int)(wid - (long)b * H);
  const int p = past[b];
  int p0 = p - window + 1; if (p0 < 0) p0 = 0;
  float* qs = sm + wib * C;
  for (int i = lane; i < C; i += 32) qs[i] = qa[((long)b * H + h) * C + i] * scale;
  __syncwarp();
  const T* rb = ring + (long)slots[b] * ring_len * C;
  float m = -INFINITY, l = 0.f, acc[ABS_MAXC];
#pragma unroll
  for (int i = 0; i < ABS_MAXC; ++i) acc[i] = 0.f;
  for (int e = p0; e <= p; e += 32) {
    const int mine = e + lane;
    float sc = -INFINITY;
    if (mine <= p) {
      const T* cr = mine == p ? cnew + (long)b * C : rb + (long)(mine % ring_len) * C;
      float d = 0.f;
      for (int i = 0; i < C; ++i) d += qs[i] * ldf(cr + i);
      sc = d;
    }
    const float mn = fmaxf(m, warp_max(sc));
    const float corr = expf(m - mn);
    const float pr = mine <= p ? expf(sc - mn) : 0.f;
    l = l * corr + warp_sum(pr);
#pragma unroll
    for (int i = 0; i < ABS_MAXC; ++i) acc[i] *= corr;
    const int cnt = min(32, p - e + 1);
    for (int k = 0; k < cnt; ++k) {
      const float pk = __shfl_sync(0xffffffffu, pr, k);
      const T* cr = (e + k) == p ? cnew + (long)b * C : rb + (long)((e + k) % ring_len) * C;
#pragma unroll
      for (int i = 0; i < ABS_MAXC; ++i) { const int c = lane + 32 * i; if (c < C) acc[i] += pk * ldf(cr + c); }
    }
    m = mn;
  }
  const float inv = 1.f / l;
#pragma unroll
  for (int i = 0; i < ABS_MAXC; ++i) { const int c = lane + 32 * i; if (c < C) out[((long)b * H + h) * C + c] = acc[i] * inv; }
}

// Split form of the same step for long windows: all heads of a sequence share its latents, so a block stages KC = 32
// of them once (plus the queries of up to 16 heads) in shared memory, computes the scores of every head against them,
// a partial softmax (max, sum) and the partial weighted sum; a second kernel merges the partials of a (sequence, head).
constexpr int KC = 32, HG = 16;

template <typename T>
__global__ void __launch_bounds__(256)
latent_decode_split_kernel(const float* __restrict__ qa, const T* __restrict__ ring, const T* __restrict__ cnew,
                           const int* __restrict__ slots, const int* __restrict__ past, float* __restrict__ part_o,
                           float* __restrict__ part_ml, int H, int C, int ring_len, int window, int nch, float scale) {
  extern __shared__ __align__(16) unsigned char smraw[];
  const int b = blockIdx.x, ch = blockIdx.y, h0 = blockIdx.z * HG;
  const int hg = min(HG, H - h0);
  const int p = past[b];
  int p0 = p - window + 1; if (p0 < 0) p0 = 0;
  const int e0 = p0 + ch * KC;
  if (e0 > p) return;                                           // the whole block leaves: no barrier is skipped
  const int cnt = min(KC, p - e0 + 1);
  const int LS = C + (sizeof(T) == 2 ? 2 : 1);                  // tile row stride: an odd number of 32-bit words
  float* sq = reinterpret_cast<float*>(smraw);                  // [HG][C]
  float* ss = sq + HG * C;                                      // [HG][KC]
  T* sl = reinterpret_cast<T*>(ss + HG * KC);                   // [KC][LS]
  const int tid = threadIdx.x;
  for (int e = tid; e < hg * C; e += 256) sq[e] = qa[((long)b * H + h0) * C + e] * scale;
  const T* rb = ring + (long)slots[b] * ring_len * C;
  for (int e = tid; e < cnt * C; e += 256) {
    const int kk = e / C, c = e - kk * C, pos = e0 + kk;
    sl[kk * LS + c] = pos == p ? cnew[(long)b * C + c] : rb[(long)(pos % ring_len) * C + c];
  }
  __syncthreads();
  const int lane = tid & 31, w = tid >> 5;
  for (int hh = w; hh < hg; hh += 8) {                          // one warp per head: lane = key
    float sc = -INFINITY;
    if (lane < cnt) {
      float d = 0.f;
      const float* qr = sq + hh * C; const T* lr = sl + lane * LS;
      for (int c = 0; c < C; ++c) d += qr[c] * ldf(lr + c);
      sc = d;
    }
    const float m = warp_max(sc);
    const float pr = lane < cnt ? expf(sc - m) : 0.f;
    const float l = warp_sum(pr);
    ss[hh * KC + lane] = pr;
    if (lane == 0) { float* ml = part_ml + (((long)b * H + h0 + hh) * nch + ch) * 2; ml[0] = m; ml[1] = l; }
  }
  __syncthreads();
  for (int c = tid; c < C; c += 256) {
    float acc[HG];
#pragma unroll
    for (int hh = 0; hh < HG; ++hh) acc[hh] = 0.f;
    for (int kk = 0; kk < cnt; ++kk) {
      const float lv = ldf(sl + kk * LS + c);
#pragma unroll
      for (int hh = 0; hh < HG; ++hh) acc[hh] += ss[hh * KC + kk] * lv;   // rows >= hg hold stale values that are not stored
    }
#pragma unroll
    for (int hh = 0; hh < HG; ++hh)
      if (hh < hg) part_o[(((long)b * H + h0 + hh) * nch + ch) * C + c] = acc[hh];
  }
}

__global__ void latent_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                           const int* __restrict__ past, float* __restrict__ out, int H, int C, int window, int nch) {
  const int b = blockIdx.x / H;
  const int p = past[b];
  int p0 = p - window + 1; if (p0 < 0) p0 = 0;
  const int used = (p - p0) / KC + 1;
  const float* ml = part_ml + (long)blockIdx.x * nch * 2;
  float M = -INFINITY;
  for (int c = 0; c < used; ++c) M = fmaxf(M, ml[2 * c]);
  float L = 0.f;
  for (int c = 0; c < used; ++c) L += expf(ml[2 * c] - M) * ml[2 * c + 1];
  for (int i = threadIdx.x; i < C; i += blockDim.x) {
    float acc = 0.f;
    for (int c = 0; c < used; ++c) acc += expf(ml[2 * c] - M) * part_o[((long)blockIdx.x * nch + c) * C + i];
    out[(long)blockIdx.x * C + i] = acc / L;
  }
}

// y[b, h*V + v] = x[b, h, v] * sigmoid(gate[b, h]) (fp32 in, T out)
template <typename T>
__global__ void head_gate_kernel(const float* __restrict__ x, const T* __restrict__ gate, long ldg, T* __restrict__ y, long ldy,
                                 long rows, int H, int V) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * H * V) return;
  const long row = idx / ((long)H * V); const int hv = (int)(idx - row * (long)H * V); const int h = hv / V;
  const float g = gate ? sigmoidf_(ldf(gate + row * ldg + h)) : 1.f;
  stf(y + row * ldy + hv, x[idx] * g);
}

inline int cdiv(long a, long b) { return (int)((a + b - 1) / b); }
inline int ok() { return (int)cudaGetLastError(); }
typedef __nv_bfloat16 bf16;

}  // namespace

#define DISPATCH(dtype, ...)                         \
  if ((dtype) == 0) { typedef float T; __VA_ARGS__; } \
  else { typedef bf16 T; __VA_ARGS__; }

extern "C" {

// x: rows of `xdtype` (0 fp32, 1 bf16); w and y: `dtype`; ids optional row gather
int lbs_rmsnorm(const void* x, long ldx, int xdtype, const int64_t* ids, const void* w, float offset, float eps, void* y, long ldy,
                int ydtype, int wdtype, long rows, int n, cudaStream_t s) {
  if (rows == 0) return 0;
  const int th = n >= 1024 ? 256 : (n >= 256 ? 128 : 64);
#define RN(TI, TW, TO) rmsnorm_kernel<TI, TW, TO><<<(unsigned)rows, th, 0, s>>>((const TI*)x, ldx, ids, (const TW*)w, offset, eps, (TO*)y, ldy, n)
  const int key = xdtype * 4 + wdtype * 2 + ydtype;
  switch (key) {
    case 0: RN(float, float, float); break;
    case 1: RN(float, float, bf16); break;
    case 2: RN(float, bf16, float); break;
    case 3: RN(float, bf16, bf16); break;
    case 4: RN(bf16, float, float); break;
    case 5: RN(bf16, float, bf16); break;
    case 6: RN(bf16, bf16, float); break;
    default: RN(bf16, bf16, bf16); break;
  }
#undef RN
  return ok();
}

int lbs_slice_act(const void* in, long ldi, int idtype, void* out, long ldo, int odtype, long rows, int n, int act, cudaStream_t s) {
  if (rows * n == 0) return 0;
  if (idtype == 1 && odtype == 1 && n % 8 == 0 && ldi % 8 == 0 && ldo % 8 == 0 && ((uintptr_t)in) % 16 == 0 && ((uintptr_t)out) % 16 == 0) {
    slice_act_vec8_kernel<<<cdiv(rows * (n / 8), 256), 256, 0, s>>>((const bf16*)in, ldi, (bf16*)out, ldo, rows, n / 8, act);
    return ok();
  }
  const int g = cdiv(rows * n, 256);
  if (idtype == 0 && odtype == 0) slice_act_kernel<float, float><<<g, 256, 0, s>>>((const float*)in, ldi, (float*)out, ldo, rows, n, act);
  else if (idtype == 0) slice_act_kernel<float, bf16><<<g, 256, 0, s>>>((const float*)in, ldi, (bf16*)out, ldo, rows, n, act);
  else if (odtype == 0) slice_act_kernel<bf16, float><<<g, 256, 0, s>>>((const bf16*)in, ldi, (float*)out, ldo, rows, n, act);
  else slice_act_kernel<bf16, bf16><<<g, 256, 0, s>>>((const bf16*)in, ldi, (bf16*)out, ldo, rows, n, act);
  return ok();
}

int lbs_short_conv(const void* in, long ldi, const void* w, void* tail, const int* tok_seq, const int* seq_off, const int* slots,
                   const int* past, void* out, long ldo, long tokens, int B, int C, int taps, int dtype, cudaStream_t s) {
  if (tokens == 0) return 0;
  const bool vec = dtype == 1 && C % 8 == 0 && ldi % 8 == 0 && ldo % 8 == 0 && taps >= 2 && taps <= 4 && ((uintptr_t)in) % 16 == 0 &&
                   ((uintptr_t)out) % 16 == 0 && ((uintptr_t)tail) % 16 == 0 && ((uintptr_t)w) % 16 == 0;
  if (vec) {
    const int g = cdiv(tokens * (C / 8), 256);
#define SC(TP)                                                                                                                   \
  short_conv_vec8_kernel<TP><<<g, 256, 0, s>>>((const bf16*)in, ldi, (const bf16*)w, (const bf16*)tail, tok_seq, seq_off, slots, past, \
                                               (bf16*)out, ldo, tokens, C)
    if (taps == 2) SC(2); else if (taps == 3) SC(3); else SC(4);
#undef SC
    conv_tail_kernel<bf16><<<cdiv((long)B * C, 256), 256, 0, s>>>((const bf16*)in, ldi, (bf16*)tail, seq_off, slots, past, B, C, taps);
    return ok();
  }
  DISPATCH(dtype, {
    short_conv_kernel<T><<<cdiv(tokens * C, 256), 256, 0, s>>>((const T*)in, ldi, (const T*)w, (const T*)tail, tok_seq, seq_off, slots,
                                                                past, (T*)out, ldo, tokens, C, taps);
    if (taps > 1)
      conv_tail_kernel<T><<<cdiv((long)B * C, 256), 256, 0, s>>>((const T*)in, ldi, (T*)tail, seq_off, slots, past, B, C, taps);
  });
  return ok();
}

// work: fp32 scratch of at least tokens * (2*KH*D + KH + H + (chan ? H*D : H)) floats
int lbs_delta_scan(const void* qkv, long ldq, int koff, int voff, const void* a, long lda, const void* bl, long ldb, const void* A_log,
                   const void* dt_bias, float* S, const int* seq_off, const int* slots, const int* past, float* out, float* work,
                   long tokens, int B, int H, int KH, int D, int V, int chan, int dtype, cudaStream_t s) {
  if (B == 0 || tokens == 0) return 0;
  if (D > 256 || H % KH != 0) return -1;
  float* qn = work;
  float* kn = qn + tokens * KH * D;
  float* kq = kn + tokens * KH * D;
  float* beta = kq + tokens * KH;
  float* g = beta + tokens * H;
  DISPATCH(dtype, delta_prep_kernel<T><<<cdiv(tokens * KH * 32, 256), 256, 0, s>>>((const T*)qkv, ldq, koff, (const T*)a, lda, (const T*)bl,
                                                                                  ldb, (const T*)A_log, (const T*)dt_bias, qn, kn, kq, g,
                                                                                  beta, tokens, H, KH, D, chan));
  const int dpt = D <= 32 ? 8 : (D <= 128 ? 16 : 32);  // rows per lane: 4 lanes per column up to D = 64, 8 lanes up to 256
  int R = 1;
  while (R * dpt < D) R <<= 1;                   // a power of two <= 8
  int VT = R <= 4 ? 64 : 32;                     // columns per block (columns are independent: more blocks per head)
  if (V < VT) VT = V;
  int threads = ((VT * R + 31) / 32) * 32;
  const int Dp = R * (dpt + 4);
  const size_t smem = sizeof(float) * ((size_t)CT * Dp * 2 + (size_t)CT * (chan ? Dp : 4) + (size_t)CT * VT + 2 * CT);
  dim3 grid((unsigned)(B * H), (unsigned)((V + VT - 1) / VT));
#define DS(TT, P)                                                                                                              \
  {                                                                                                                            \
    if (smem > 48 * 1024) cudaFuncSetAttribute(delta_scan_kernel<TT, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    delta_scan_kernel<TT, P><<<grid, threads, smem, s>>>((const TT*)qkv, ldq, voff, qn, kn, kq, g, beta, S, seq_off, slots, past, out, \
                                                        H, KH, D, V, R, VT, chan);                                              \
  }
  if (dtype == 0) { if (dpt == 8) DS(float, 8) else if (dpt == 16) DS(float, 16) else DS(float, 32) }
  else { if (dpt == 8) DS(bf16, 8) else if (dpt == 16) DS(bf16, 16) else DS(bf16, 32) }
#undef DS
  return ok();
}

int lbs_gated_rmsnorm(const float* o, const void* gate, long ldg, const void* w, float eps, int act, void* y, long ldy, long rows,
                      int H, int V, int dtype, cudaStream_t s) {
  if (rows == 0) return 0;
  DISPATCH(dtype, gated_rmsnorm_kernel<T><<<cdiv(rows * H * 32, 256), 256, 0, s>>>(o, (const T*)gate, ldg, (const T*)w, eps, act,
                                                                                    (T*)y, ldy, rows, H, V));
  return ok();
}

int lbs_latent_gather(const void* ring, const void* cnew, const int* ext_seq, const int* ext_off, const int* seq_off, const int* slots,
                      const int* past, void* ext, long rows, int C, int ring_len, int dtype, cudaStream_t s) {
  if (rows == 0) return 0;
  DISPATCH(dtype, latent_gather_kernel<T><<<cdiv(rows * C, 256), 256, 0, s>>>((const T*)ring, (const T*)cnew, ext_seq, ext_off, seq_off,
                                                                               slots, past, (T*)ext, rows, C, ring_len));
  return ok();
}

int lbs_latent_write(void* ring, const void* cnew, const int* tok_seq, const int* seq_off, const int* slots, const int* past,
                     long tokens, int C, int ring_len, int dtype, cudaStream_t s) {
  if (tokens == 0) return 0;
  DISPATCH(dtype, latent_write_kernel<T><<<cdiv(tokens * C, 256), 256, 0, s>>>((T*)ring, (const T*)cnew, tok_seq, seq_off, slots, past,
                                                                                tokens, C, ring_len));
  return ok();
}

int lbs_window_attention(const void* q, long ldq, const void* kv, long ldkv, const void* gate, long ldg, const int* tok_seq,
                         const int* seq_off, const int* ext_off, const int* qt_seq, const int* qt_start, int n_qtiles, void* y,
                         long ldy, long tokens, int H, int D, int V, int window, float scale, int dtype, cudaStream_t s) {
  if (tokens == 0) return 0;
  if (V > 32 * ATT_MAXV) return -1;
  const bool aligned = (ldkv % 8 == 0) && (ldq % 2 == 0) && (ldy % 2 == 0) && (((uintptr_t)kv) % 16 == 0) &&
                       (((uintptr_t)q) % 4 == 0) && (((uintptr_t)y) % 4 == 0);
  if (dtype == 1 && qt_seq != nullptr && n_qtiles > 0 && aligned) {
    dim3 grid((unsigned)n_qtiles, (unsigned)H);
#define WA(DD, VV)                                                                                                        \
  if (D == DD && V == VV) {                                                                                                \
    window_attention_mma_kernel<DD, VV><<<grid, 128, 0, s>>>((const bf16*)q, ldq, (const bf16*)kv, ldkv, (const bf16*)gate, ldg, \
                                                             qt_seq, qt_start, seq_off, ext_off, (bf16*)y, ldy, H, window, scale); \
    return ok();                                                                                                           \
  }
    WA(32, 32) WA(64, 64) WA(128, 128) WA(64, 128) WA(128, 64) WA(32, 64) WA(64, 32)
#undef WA
  }
  const int warps = 4;
  const size_t smem = sizeof(float) * warps * D;
  DISPATCH(dtype, window_attention_kernel<T><<<cdiv(tokens * H, warps), warps * 32, smem, s>>>(
                      (const T*)q, ldq, (const T*)kv, ldkv, (const T*)gate, ldg, tok_seq, seq_off, ext_off, (T*)y, ldy, tokens, H, D, V,
                      window, scale));
  return ok();
}

// part_o: [B, H, nch, C] fp32 and part_ml: [B, H, nch, 2] fp32 workspaces with nch = ceil(window / 32), or null: then (and for
// windows of at most 64 positions) one warp per (sequence, head) does the whole window
int lbs_latent_decode(const float* qa, const void* ring, const void* cnew, const int* slots, const int* past, float* out,
                      float* part_o, float* part_ml, int B, int H, int C, int ring_len, int window, float scale, int dtype,
                      cudaStream_t s) {
  if (B == 0) return 0;
  if (part_o != nullptr && part_ml != nullptr && window > 64) {
    const int nch = (window + KC - 1) / KC;
    const int hg = H < HG ? H : HG;
    const size_t esz = dtype == 0 ? 4 : 2;
    const size_t smem = sizeof(float) * ((size_t)HG * C + HG * KC) + esz * KC * (C + (dtype == 0 ? 1 : 2));
    (void)hg;
    if (smem <= 200 * 1024) {
      dim3 grid((unsigned)B, (unsigned)nch, (unsigned)((H + HG - 1) / HG));
      DISPATCH(dtype, {
        if (smem > 48 * 1024) cudaFuncSetAttribute(latent_decode_split_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        latent_decode_split_kernel<T><<<grid, 256, smem, s>>>(qa, (const T*)ring, (const T*)cnew, slots, past, part_o, part_ml, H, C,
                                                              ring_len, window, nch, scale);
      });
      latent_decode_merge_kernel<<<B * H, 128, 0, s>>>(part_o, part_ml, past, out, H, C, window, nch);
      return ok();
    }
  }
  if (C > 32 * ABS_MAXC) return -1;
  const int warps = 4;
  const size_t smem = sizeof(float) * warps * C;
  DISPATCH(dtype, latent_decode_kernel<T><<<cdiv((long)B * H, warps), warps * 32, smem, s>>>(qa, (const T*)ring, (const T*)cnew, slots,
                                                                                              past, out, B, H, C, ring_len, window, scale));
  return ok();
}

int lbs_head_gate(const float* x, const void* gate, long ldg, void* y, long ldy, long rows, int H, int V, int dtype, cudaStream_t s) {
  if (rows == 0) return 0;
  DISPATCH(dtype, head_gate_kernel<T><<<cdiv(rows * H * V, 256), 256, 0, s>>>(x, (const T*)gate, ldg, (T*)y, ldy, rows, H, V));
  return ok();
}

}  // extern "C"
