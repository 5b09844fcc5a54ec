// Ragged sequence-mixer kernels: sum + RMS norm of an fp32 residual stream, short causal convolutions with carried inputs, the fused
// front half of a convolved-projection attention layer (convolution + row-wide q/k norm + partial interleaved rotation + paged cache
// write), soft-capped kept-prefix sliding-window attention over the paged cache, the Mamba-2 recurrence with a carried fp32 state,
// grouped RMS norm and the clamped gate product.  Norms, softmax, decays, step sizes and states are fp32; activations are bf16 or fp32
// (template parameter).  This file is compiled WITHOUT fast-math: tanh / exp / divisions are the accurate ones.
#include <cuda_bf16.h>
#include <math.h>

#include "common.cuh"
#include "seqmix.h"

namespace nxdi {
namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// sum over the block; every thread gets the result.  `red` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : 0.f;
  return warp_sum(t);
}

__device__ __forceinline__ float sigmoidf_acc(float x) { return 1.f / (1.f + expf(-x)); }

// ---- out = rms_unit(alpha * x + y) * (offset + w) ---------------------------------------------------------------------------
template <typename TY>
__global__ void __launch_bounds__(256) scaled_add_rmsnorm_kernel(const float* __restrict__ x, const TY* __restrict__ y,
                                                                 const float* __restrict__ w, float* __restrict__ out,
                                                                 __nv_bfloat16* __restrict__ out_lp, int W, float alpha, float eps,
                                                                 float offset) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const float* xr = x + row * W;
  const TY* yr = y ? y + row * W : nullptr;
  float ss = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float s = alpha * xr[c] + (yr ? ldf(yr + c) : 0.f);
    ss += s * s;
  }
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / (float)W + eps);
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float s = alpha * xr[c] + (yr ? ldf(yr + c) : 0.f);
    float o = s * r * (w ? (w[c] + offset) : 1.f);
    out[row * W + c] = o;
    if (out_lp) out_lp[row * W + c] = __float2bfloat16_rn(o);
  }
}

// ---- short causal convolution with carried inputs ----------------------------------------------------------------------------
// input at window index i (i = t - K + 1 + j): i >= 0 -> u[b, i]; i < 0 -> carried row K - 1 + i of the line (zero when ctx == 0)
template <typename T>
__device__ __forceinline__ float conv_input(const T* u_row0, long long u_st, const T* st_line, int C, int K, int i, int c, bool has_ctx) {
  if (i >= 0) return ldf(u_row0 + (long long)i * u_st + c);
  return has_ctx ? ldf(st_line + (long long)(K - 1 + i) * C + c) : 0.f;
}

template <typename T>
__global__ void __launch_bounds__(256) short_conv_kernel(const T* __restrict__ u, long long u_sb, long long u_st,
                                                         const float* __restrict__ w, const float* __restrict__ bias,
                                                         const T* __restrict__ state, const int* __restrict__ lines,
                                                         const int* __restrict__ ctx_len, const int* __restrict__ q_len,
                                                         float* __restrict__ y, int T_, int C, int K, int silu) {
  const int b = blockIdx.z, t = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C || t >= q_len[b]) return;
  const bool has_ctx = ctx_len[b] > 0;
  const T* u0 = u + (long long)b * u_sb;
  const T* sl = state + (long long)lines[b] * (K - 1) * C;
  float acc = bias ? bias[c] : 0.f;
  for (int j = 0; j < K; ++j) acc += w[(long long)c * K + j] * conv_input(u0, u_st, sl, C, K, t - K + 1 + j, c, has_ctx);
  if (silu) acc = acc * sigmoidf_acc(acc);
  y[((long long)b * T_ + t) * C + c] = acc;
}

template <typename T>
__global__ void __launch_bounds__(256) short_conv_update_kernel(const T* __restrict__ u, long long u_sb, long long u_st, T* __restrict__ state,
                                                                const int* __restrict__ lines, const int* __restrict__ ctx_len,
                                                                const int* __restrict__ q_len, int C, int K) {
  const int b = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  const int n = q_len[b];
  if (c >= C || n <= 0) return;
  const bool has_ctx = ctx_len[b] > 0;
  const T* u0 = u + (long long)b * u_sb;
  T* sl = state + (long long)lines[b] * (K - 1) * C;
  float keep[SEQMIX_MAX_TAPS];
  // new row j = input at window index n - (K - 1) + j
#pragma unroll
  for (int j = 0; j < SEQMIX_MAX_TAPS - 1; ++j)
    if (j < K - 1) keep[j] = conv_input(u0, u_st, sl, C, K, n - (K - 1) + j, c, has_ctx);
#pragma unroll
  for (int j = 0; j < SEQMIX_MAX_TAPS - 1; ++j)
    if (j < K - 1) stf(sl + (long long)j * C + c, keep[j]);
}

// ---- convolution + row-wide q / k norm + partial interleaved rotation + paged cache write -------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) conv_qknorm_rope_append_kernel(ConvQkParams p) {
  extern __shared__ float buf[];      // [Cq + Ck + Cv] convolved row
  __shared__ float red[32];
  const int b = blockIdx.y, t = blockIdx.x;
  if (t >= p.q_len[b]) return;
  const int Cq = p.n_q * p.D, Ck = p.n_kv * p.D, Cv = p.n_kv * p.Dv, C = Cq + Ck + Cv, K = p.K;
  const bool has_ctx = p.ctx_len[b] > 0;
  const T* u0 = (const T*)p.p + (long long)b * p.p_sb;
  const T* sl = (const T*)p.state + (long long)p.lines[b] * (K - 1) * C;
  float sq = 0.f, sk = 0.f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < K; ++j) acc += p.conv_w[(long long)c * K + j] * conv_input(u0, p.p_st, sl, C, K, t - K + 1 + j, c, has_ctx);
    buf[c] = acc;
    if (c < Cq) sq += acc * acc;
    else if (c < Cq + Ck) sk += acc * acc;
  }
  sq = block_sum(sq, red);
  sk = block_sum(sk, red);
  const float rq = 1.f / sqrtf(sq / (float)Cq + p.eps);
  const float rk = Ck ? 1.f / sqrtf(sk / (float)Ck + p.eps) : 0.f;
  const long long tok = (long long)b * p.T + t;
  const float* cs = p.cos + tok * (p.R / 2);
  const float* sn = p.sin + tok * (p.R / 2);
  const int pos = p.ctx_len[b] + t;
  long long slot = 0;
  if (p.n_kv) slot = (long long)p.block_table[(long long)b * p.max_blocks + pos / p.page] * p.page + pos % p.page;
  T* qo = (T*)p.q_out + tok * Cq;
  T* ko = (T*)p.k_cache + slot * Ck;
  T* vo = (T*)p.v_cache + slot * Cv;
  for (int c = threadIdx.x; c < Cq + Ck; c += blockDim.x) {
    const bool isq = c < Cq;
    const int cc = isq ? c : c - Cq;
    const float r = isq ? rq : rk;
    const float* nw = isq ? p.q_norm_w : p.k_norm_w;
    const int d = cc % p.D;
    float self = buf[c] * r * nw[cc];
    if (d < p.R) {
      const float other = buf[c ^ 1] * r * nw[cc ^ 1];
      const float co = cs[d >> 1], si = sn[d >> 1];
      self = (d & 1) ? (self * co + other * si) : (self * co - other * si);
    }
    stf((isq ? qo : ko) + cc, self);
  }
  for (int c = threadIdx.x; c < Cv; c += blockDim.x) stf(vo + c, buf[Cq + Ck + c]);
}

// ---- soft-capped kept-prefix sliding-window attention over the paged cache ---------------------------------------------------
template <typename T> struct Vec;                     // 16-byte vectors of the activation type
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<__nv_bfloat16> { static constexpr int N = 8; };

template <typename T>
__device__ __forceinline__ float dot_row(const float* qs, const T* k, int D, bool vec_ok) {
  float s = 0.f;
  if (vec_ok) {
    constexpr int N = Vec<T>::N;
    for (int d = 0; d < D; d += N) {
      const uint4 raw = *reinterpret_cast<const uint4*>(k + d);
      if constexpr (N == 4) {
        s += qs[d] * __uint_as_float(raw.x) + qs[d + 1] * __uint_as_float(raw.y) + qs[d + 2] * __uint_as_float(raw.z) +
             qs[d + 3] * __uint_as_float(raw.w);
      } else {
        s += qs[d] * bf16lo(raw.x) + qs[d + 1] * bf16hi(raw.x) + qs[d + 2] * bf16lo(raw.y) + qs[d + 3] * bf16hi(raw.y) +
             qs[d + 4] * bf16lo(raw.z) + qs[d + 5] * bf16hi(raw.z) + qs[d + 6] * bf16lo(raw.w) + qs[d + 7] * bf16hi(raw.w);
      }
    }
  } else {
    for (int d = 0; d < D; ++d) s += qs[d] * ldf(k + d);
  }
  return s;
}

constexpr int ATT_WARPS = 4;
constexpr int ATT_VPL = SEQMIX_MAX_VDIM / 32;      // value channels per lane

// SPLIT = false: warp w of a block owns query blockIdx.x * 4 + w.  SPLIT = true: the four warps share query blockIdx.x, warp w takes
// key chunks w, w + 4, ... and the partial (max, sum, acc) are merged through shared memory (few queries, long ranges: decode).
template <typename T, bool SPLIT>
__global__ void __launch_bounds__(ATT_WARPS * 32) paged_window_attention_kernel(WindowAttnParams p) {
  extern __shared__ float smem[];      // [ATT_WARPS][D] scaled queries, then (SPLIT) [ATT_WARPS][Dv + 2] partials
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long nq = (long long)p.B * p.T * p.Hq;
  const long long qi = SPLIT ? (long long)blockIdx.x : (long long)blockIdx.x * ATT_WARPS + warp;
  const bool in_range = qi < nq;
  const int h = in_range ? (int)(qi % p.Hq) : 0;
  const long long tok = in_range ? qi / p.Hq : 0;
  const int b = (int)(tok / p.T), t = (int)(tok % p.T);
  const bool live = in_range && t < p.q_len[b];
  if (!SPLIT && !live) return;
  if (SPLIT && !live) return;          // uniform over the block: all warps share the query
  const int D = p.D, Dv = p.Dv, g = h / (p.Hq / p.G);
  float* qs = smem + warp * D;
  const T* qrow = (const T*)p.q + qi * D;
  for (int d = lane; d < D; d += 32) qs[d] = ldf(qrow + d) * p.scale;
  __syncwarp();
  const int pos = p.ctx_len[b] + t;
  const int lo = p.window > 0 ? max(pos - p.window + 1, 0) : 0;
  const int nA = p.window > 0 ? min(p.keep_first, lo) : 0;       // kept first tokens that the window no longer covers
  const int n = nA + (pos - lo + 1);
  const int* table = p.block_table + (long long)b * p.max_blocks;
  const bool kvec = ((D * (int)sizeof(T)) % 16) == 0;
  const T* kc = (const T*)p.k_cache;
  const T* vc = (const T*)p.v_cache;
  float m = -INFINITY, l = 0.f, acc[ATT_VPL];
#pragma unroll
  for (int i = 0; i < ATT_VPL; ++i) acc[i] = 0.f;
  const int nchunks = (n + 31) / 32;
  for (int ch = SPLIT ? warp : 0; ch < nchunks; ch += SPLIT ? ATT_WARPS : 1) {
    const int idx = ch * 32 + lane;
    float s = -INFINITY;
    long long row = 0;
    if (idx < n) {
      const int j = idx < nA ? idx : lo + (idx - nA);
      row = ((long long)table[j / p.page] * p.page + j % p.page) * p.G + g;
      s = dot_row(qs, kc + row * D, D, kvec);
      if (p.softcap > 0.f) s = p.softcap * tanhf(s / p.softcap);
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);          // m = -inf on the first chunk: exp(-inf) = 0
    const float pj = idx < n ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(pj);
#pragma unroll
    for (int i = 0; i < ATT_VPL; ++i) acc[i] *= corr;
    m = m_new;
    const int cnt = min(32, n - ch * 32);
    for (int jj = 0; jj < cnt; ++jj) {
      const float pw = __shfl_sync(0xffffffffu, pj, jj);
      const long long r = __shfl_sync(0xffffffffu, row, jj);
      const T* vrow = vc + r * Dv;
#pragma unroll
      for (int i = 0; i < ATT_VPL; ++i) {
        const int dv = lane + 32 * i;
        if (dv < Dv) acc[i] += pw * ldf(vrow + dv);
      }
    }
  }
  if (SPLIT) {
    float* part = smem + ATT_WARPS * D + warp * (Dv + 2);
#pragma unroll
    for (int i = 0; i < ATT_VPL; ++i) {
      const int dv = lane + 32 * i;
      if (dv < Dv) part[dv] = acc[i];
    }
    if (lane == 0) { part[Dv] = m; part[Dv + 1] = l; }
    __syncthreads();
    if (warp != 0) return;
    float M = -INFINITY;
    for (int w = 0; w < ATT_WARPS; ++w) M = fmaxf(M, smem[ATT_WARPS * D + w * (Dv + 2) + Dv]);
    l = 0.f;
#pragma unroll
    for (int i = 0; i < ATT_VPL; ++i) acc[i] = 0.f;
    for (int w = 0; w < ATT_WARPS; ++w) {
      const float* pw = smem + ATT_WARPS * D + w * (Dv + 2);
      const float f = pw[Dv] == -INFINITY ? 0.f : expf(pw[Dv] - M);
      l += pw[Dv + 1] * f;
#pragma unroll
      for (int i = 0; i < ATT_VPL; ++i) {
        const int dv = lane + 32 * i;
        if (dv < Dv) acc[i] += pw[dv] * f;
      }
    }
  }
  const float inv = 1.f / l;
  T* orow = (T*)p.out + qi * Dv;
  const T* grow = p.gate ? (const T*)p.gate + (long long)b * p.g_sb + (long long)t * p.g_st + (long long)h * Dv : nullptr;
#pragma unroll
  for (int i = 0; i < ATT_VPL; ++i) {
    const int dv = lane + 32 * i;
    if (dv < Dv) {
      float o = acc[i] * inv;
      if (grow) o *= sigmoidf_acc(ldf(grow + dv));
      stf(orow + dv, o);
    }
  }
}

// ---- Mamba-2 recurrence with a carried state ----------------------------------------------------------------------------------
constexpr int SCAN_PT = 16;      // head channels per block
constexpr int SCAN_NS = 8;       // lanes that split the state axis for one channel
constexpr int SCAN_TT = 16;      // time steps staged per round
constexpr int SCAN_NPT = SEQMIX_MAX_STATE / SCAN_NS;

template <typename T>
__global__ void __launch_bounds__(SCAN_PT* SCAN_NS) ssd_scan_kernel(SsdScanParams p) {
  extern __shared__ float sm[];
  const int N = p.N, P = p.P;
  float* Bs = sm;                          // [TT][N]
  float* Cs = Bs + SCAN_TT * N;            // [TT][N]
  float* xs = Cs + SCAN_TT * N;            // [TT][PT]
  float* ys = xs + SCAN_TT * SCAN_PT;      // [TT][PT]
  float* dts = ys + SCAN_TT * SCAN_PT;     // [TT]
  float* dAs = dts + SCAN_TT;              // [TT]
  const int b = blockIdx.z, h = blockIdx.y, p0 = blockIdx.x * SCAN_PT;
  const int n_tok = p.q_len[b];
  if (n_tok <= 0) return;
  const int tid = threadIdx.x, pl = tid / SCAN_NS, ns = tid % SCAN_NS;
  const int pc = p0 + pl;                  // this thread's head channel
  const bool pok = pc < P;
  const int g = h / (p.nh / p.G);
  const int inner = p.nh * P, Cd = inner + 2 * p.G * N;
  float* Sg = p.state + ((long long)p.lines[b] * p.nh + h) * N * P;
  float S[SCAN_NPT];
  const bool has_ctx = p.ctx_len[b] > 0;
#pragma unroll
  for (int i = 0; i < SCAN_NPT; ++i) {
    const int n = ns + SCAN_NS * i;
    S[i] = (has_ctx && pok && n < N) ? Sg[(long long)n * P + pc] : 0.f;
  }
  const float negA = -expf(p.A_log[h]), dtb = p.dt_bias[h], Dh = p.D_skip[h];
  const float* xrow = p.xBC + (long long)b * p.T * Cd;
  const T* dtp = (const T*)p.dt_raw + (long long)b * p.dt_sb + h;
  for (int t0 = 0; t0 < n_tok; t0 += SCAN_TT) {
    const int tt = min(SCAN_TT, n_tok - t0);
    __syncthreads();
    for (int i = tid; i < tt * N; i += blockDim.x) {
      const int t = i / N, n = i % N;
      const float* r = xrow + (long long)(t0 + t) * Cd + inner + g * N + n;
      Bs[t * N + n] = r[0];
      Cs[t * N + n] = r[p.G * N];
    }
    for (int i = tid; i < tt * SCAN_PT; i += blockDim.x) {
      const int t = i / SCAN_PT, c = p0 + i % SCAN_PT;
      xs[i] = c < P ? xrow[(long long)(t0 + t) * Cd + h * P + c] : 0.f;
    }
    if (tid < tt) {
      const float v = ldf(dtp + (long long)(t0 + tid) * p.dt_st) + dtb;
      const float dt = v > 20.f ? v : log1pf(expf(v));
      dts[tid] = dt;
      dAs[tid] = expf(negA * dt);
    }
    __syncthreads();
    for (int t = 0; t < tt; ++t) {
      const float dA = dAs[t], dx = dts[t] * xs[t * SCAN_PT + pl];
      const float* Bt = Bs + t * N;
      const float* Ct = Cs + t * N;
      float y = 0.f;
#pragma unroll
      for (int i = 0; i < SCAN_NPT; ++i) {
        const int n = ns + SCAN_NS * i;
        if (n < N) {
          S[i] = dA * S[i] + dx * Bt[n];
          y += S[i] * Ct[n];
        }
      }
#pragma unroll
      for (int o = SCAN_NS / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
      if (ns == 0) ys[t * SCAN_PT + pl] = y + Dh * xs[t * SCAN_PT + pl];
    }
    __syncthreads();
    for (int i = tid; i < tt * SCAN_PT; i += blockDim.x) {
      const int t = i / SCAN_PT, c = p0 + i % SCAN_PT;
      if (c < P) {
        const long long tok = (long long)b * p.T + t0 + t;
        const float zv = ldf((const T*)p.z + (long long)b * p.z_sb + (long long)(t0 + t) * p.z_st + h * P + c);
        p.y[tok * inner + h * P + c] = ys[i] * (zv * sigmoidf_acc(zv));
      }
    }
  }
#pragma unroll
  for (int i = 0; i < SCAN_NPT; ++i) {
    const int n = ns + SCAN_NS * i;
    if (pok && n < N) Sg[(long long)n * P + pc] = S[i];
  }
}

// ---- grouped RMS norm ---------------------------------------------------------------------------------------------------------
template <typename TO>
__global__ void __launch_bounds__(256) group_rmsnorm_kernel(const float* __restrict__ y, const float* __restrict__ w, TO* __restrict__ out,
                                                            int W, int gw, float eps) {
  __shared__ float red[32];
  const long long base = (long long)blockIdx.y * W + (long long)blockIdx.x * gw;
  float ss = 0.f;
  for (int c = threadIdx.x; c < gw; c += blockDim.x) {
    const float v = y[base + c];
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / (float)gw + eps);
  for (int c = threadIdx.x; c < gw; c += blockDim.x) stf(out + base + c, y[base + c] * r * w[blockIdx.x * gw + c]);
}

// ---- clamped gate product -----------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) clamped_glu_kernel(const T* __restrict__ gu, T* __restrict__ out, long long rows, int F, float limit,
                                                          float alpha) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * F) return;
  const long long r = i / F;
  const int c = (int)(i % F);
  const float g = fminf(ldf(gu + r * 2 * F + c), limit);
  const float u = fminf(fmaxf(ldf(gu + r * 2 * F + F + c), -limit), limit);
  stf(out + i, g * sigmoidf_acc(alpha * g) * (u + 1.f));
}

template <typename K>
void opt_in_smem(K kernel, size_t bytes) {
  if (bytes > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

}  // namespace

void scaled_add_rmsnorm_launch(const float* x, const void* y, bool y_lp, const float* w, float* out, void* out_lp, int rows, int W,
                               float alpha, float eps, float offset, cudaStream_t st) {
  if (rows <= 0) return;
  if (y_lp)
    scaled_add_rmsnorm_kernel<__nv_bfloat16><<<rows, 256, 0, st>>>(x, (const __nv_bfloat16*)y, w, out, (__nv_bfloat16*)out_lp, W, alpha, eps, offset);
  else
    scaled_add_rmsnorm_kernel<float><<<rows, 256, 0, st>>>(x, (const float*)y, w, out, (__nv_bfloat16*)out_lp, W, alpha, eps, offset);
}

void short_conv_launch(const void* u, long long u_sb, long long u_st, const float* w, const float* bias, const void* state,
                       const int* lines, const int* ctx_len, const int* q_len, float* y, int B, int T, int C, int K, bool silu, bool lp,
                       cudaStream_t st) {
  if (B <= 0 || T <= 0) return;
  dim3 grid((C + 255) / 256, T, B);
  if (lp)
    short_conv_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)u, u_sb, u_st, w, bias, (const __nv_bfloat16*)state, lines,
                                                           ctx_len, q_len, y, T, C, K, silu);
  else
    short_conv_kernel<float><<<grid, 256, 0, st>>>((const float*)u, u_sb, u_st, w, bias, (const float*)state, lines, ctx_len, q_len, y, T, C, K, silu);
}

void short_conv_update_launch(const void* u, long long u_sb, long long u_st, void* state, const int* lines, const int* ctx_len,
                              const int* q_len, int B, int T, int C, int K, bool lp, cudaStream_t st) {
  if (B <= 0 || K <= 1) return;
  dim3 grid((C + 255) / 256, B);
  if (lp)
    short_conv_update_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)u, u_sb, u_st, (__nv_bfloat16*)state, lines, ctx_len, q_len, C, K);
  else
    short_conv_update_kernel<float><<<grid, 256, 0, st>>>((const float*)u, u_sb, u_st, (float*)state, lines, ctx_len, q_len, C, K);
}

void conv_qknorm_rope_append_launch(const ConvQkParams& p, bool lp, cudaStream_t st) {
  if (p.B <= 0 || p.T <= 0) return;
  const size_t smem = sizeof(float) * (size_t)(p.n_q * p.D + p.n_kv * (p.D + p.Dv));
  dim3 grid(p.T, p.B);
  if (lp) {
    opt_in_smem(conv_qknorm_rope_append_kernel<__nv_bfloat16>, smem);
    conv_qknorm_rope_append_kernel<__nv_bfloat16><<<grid, 256, smem, st>>>(p);
  } else {
    opt_in_smem(conv_qknorm_rope_append_kernel<float>, smem);
    conv_qknorm_rope_append_kernel<float><<<grid, 256, smem, st>>>(p);
  }
}

void paged_window_attention_launch(const WindowAttnParams& p, bool lp, cudaStream_t st) {
  const long long nq = (long long)p.B * p.T * p.Hq;
  if (nq <= 0) return;
  // few queries (decode steps): one block per query, its warps split the keys; otherwise one warp per query
  const bool split = nq <= 2LL * kNumSMs * 4;
  const size_t smem = sizeof(float) * (size_t)(ATT_WARPS * p.D + (split ? ATT_WARPS * (p.Dv + 2) : 0));
  const unsigned grid = (unsigned)(split ? nq : (nq + ATT_WARPS - 1) / ATT_WARPS);
  auto go = [&](auto kernel) {
    opt_in_smem(kernel, smem);
    kernel<<<grid, ATT_WARPS * 32, smem, st>>>(p);
  };
  if (lp) {
    if (split) go(paged_window_attention_kernel<__nv_bfloat16, true>); else go(paged_window_attention_kernel<__nv_bfloat16, false>);
  } else {
    if (split) go(paged_window_attention_kernel<float, true>); else go(paged_window_attention_kernel<float, false>);
  }
}

void ssd_scan_launch(const SsdScanParams& p, bool lp, cudaStream_t st) {
  if (p.B <= 0 || p.T <= 0) return;
  const size_t smem = sizeof(float) * (size_t)(2 * SCAN_TT * p.N + 2 * SCAN_TT * SCAN_PT + 2 * SCAN_TT);
  dim3 grid((p.P + SCAN_PT - 1) / SCAN_PT, p.nh, p.B);
  if (lp) {
    opt_in_smem(ssd_scan_kernel<__nv_bfloat16>, smem);
    ssd_scan_kernel<__nv_bfloat16><<<grid, SCAN_PT * SCAN_NS, smem, st>>>(p);
  } else {
    opt_in_smem(ssd_scan_kernel<float>, smem);
    ssd_scan_kernel<float><<<grid, SCAN_PT * SCAN_NS, smem, st>>>(p);
  }
}

void group_rmsnorm_launch(const float* y, const float* w, void* out, bool out_lp, int rows, int W, int groups, float eps, cudaStream_t st) {
  if (rows <= 0) return;
  dim3 grid(groups, rows);
  if (out_lp)
    group_rmsnorm_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(y, w, (__nv_bfloat16*)out, W, W / groups, eps);
  else
    group_rmsnorm_kernel<float><<<grid, 256, 0, st>>>(y, w, (float*)out, W, W / groups, eps);
}

void clamped_glu_launch(const void* gu, void* out, long long rows, int F, float limit, float alpha, bool lp, cudaStream_t st) {
  const long long n = rows * F;
  if (n <= 0) return;
  const unsigned grid = (unsigned)((n + 255) / 256);
  if (lp)
    clamped_glu_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, rows, F, limit, alpha);
  else
    clamped_glu_kernel<float><<<grid, 256, 0, st>>>((const float*)gu, (float*)out, rows, F, limit, alpha);
}

}  // namespace nxdi
