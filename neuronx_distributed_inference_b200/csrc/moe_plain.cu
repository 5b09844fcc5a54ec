// Two-matrix experts y = W_down act(W_up x) for activations in bf16 or fp32 and for any sizes: the CUDA-core companion of the grouped
// tcgen05 path (moe_grouped.cu), which needs bf16 and sizes in multiples of 64.  The permutation is the same one (moe_plan_kernel:
// every expert's rows padded to whole 128-row tiles, static row bound, no host synchronisation):
//
//   gather    xp[row] = x[token(row)], zero rows for padding
//   GEMM 1    h = act(xp W_up[e]^T)       64 x 64 output tiles, fp32 accumulation, the expert of a tile from the tile table
//   GEMM 2    y = h W_down[e]^T
//   combine   out[token] = sum_slot affinity * y[pos[token, slot]]     (fp32, fixed slot order)
//
// and for a handful of tokens (decode steps) two weight-streaming kernels without any permutation: one warp per (entry, hidden unit),
// then one warp per (token, output channel) that walks the token's chosen experts.  Compiled WITHOUT fast-math: the fp32 instantiation
// is the exact-arithmetic path.
#include <cuda_bf16.h>

#include <stdexcept>
#include <type_traits>

#include "common.cuh"
#include "seqmix.h"

namespace nxdi {
namespace {

template <typename T> __device__ __forceinline__ float ldx(const T* p);
template <> __device__ __forceinline__ float ldx<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldx<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stx(T* p, float v);
template <> __device__ __forceinline__ void stx<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stx<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float act_apply(int act, float v) {
  switch (act) {
    case 1: return fmaxf(v, 0.f);
    case 2: { const float r = fmaxf(v, 0.f); return r * r; }
    case 3: return v / (1.f + expf(-v));
    case 4: return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    default: return v;
  }
}

template <typename T>
__global__ void __launch_bounds__(128) gather_kernel(const T* __restrict__ x, const int* __restrict__ row_entry,
                                                     const int* __restrict__ tile_expert, T* __restrict__ xp, int H, int k) {
  const int r = blockIdx.x;
  if (tile_expert[r >> 7] < 0) return;
  const int ent = row_entry[r];
  T* dst = xp + (size_t)r * H;
  if (ent < 0) {
    for (int c = threadIdx.x; c < H; c += 128) stx(dst + c, 0.f);
    return;
  }
  const T* src = x + (size_t)(ent / k) * H;
  for (int c = threadIdx.x; c < H; c += 128) dst[c] = src[c];
}

// C[r, n] = act(sum_k A[r, k] * W[e, n, k]); block = 64 x 64 outputs, 256 threads x (4 x 4), k in slices of 16
constexpr int PT = 64, PK = 16;
template <typename T>
__global__ void __launch_bounds__(256) grouped_gemm_kernel(const T* __restrict__ A, const T* __restrict__ W, T* __restrict__ C, int N, int K,
                                                           int act, const int* __restrict__ tile_expert) {
  const int r0 = blockIdx.y * PT, n0 = blockIdx.x * PT;
  const int e = tile_expert[r0 >> 7];
  if (e < 0) return;
  __shared__ float As[PK][PT + 1], Ws[PK][PT + 1];
  const T* Wb = W + (size_t)e * N * K;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += PK) {
    for (int i = threadIdx.x; i < PT * PK; i += 256) {
      const int rr = i / PK, kk = i % PK;
      const bool ink = k0 + kk < K;
      As[kk][rr] = ink ? ldx(A + (size_t)(r0 + rr) * K + k0 + kk) : 0.f;
      Ws[kk][rr] = (ink && n0 + rr < N) ? ldx(Wb + (size_t)(n0 + rr) * K + k0 + kk) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < PK; ++kk) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = As[kk][ty * 4 + i]; w[i] = Ws[kk][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) stx(C + (size_t)(r0 + ty * 4 + i) * N + n, act_apply(act, acc[i][j]));
    }
}

template <typename T>
__global__ void __launch_bounds__(128) combine_kernel(const T* __restrict__ y, const float* __restrict__ topk_w, const int* __restrict__ pos,
                                                      T* __restrict__ out, int H, int k) {
  const int tok = blockIdx.x;
  __shared__ int s_pos[64];
  __shared__ float s_w[64];
  if ((int)threadIdx.x < k) {
    s_pos[threadIdx.x] = pos[(size_t)tok * k + threadIdx.x];
    s_w[threadIdx.x] = topk_w[(size_t)tok * k + threadIdx.x];
  }
  __syncthreads();
  for (int c = threadIdx.x; c < H; c += 128) {
    float f = 0.f;
    for (int s = 0; s < k; ++s)
      if (s_pos[s] >= 0) f += s_w[s] * ldx(y + (size_t)s_pos[s] * H + c);
    stx(out + (size_t)tok * H + c, f);
  }
}

// dot product of two dense rows by one warp (every lane gets the sum); 16-byte loads when both rows allow them
template <typename T>
__device__ __forceinline__ float warp_dot(const T* a, const T* b, int n, int lane) {
  constexpr int V = 16 / (int)sizeof(T);
  float s = 0.f;
  if (n % V == 0 && (((uintptr_t)a | (uintptr_t)b) & 15) == 0) {
    for (int c = lane * V; c < n; c += 32 * V) {
      const uint4 ua = *reinterpret_cast<const uint4*>(a + c), ub = __ldg(reinterpret_cast<const uint4*>(b + c));
      if constexpr (V == 4) {
        s = fmaf(__uint_as_float(ua.x), __uint_as_float(ub.x), s); s = fmaf(__uint_as_float(ua.y), __uint_as_float(ub.y), s);
        s = fmaf(__uint_as_float(ua.z), __uint_as_float(ub.z), s); s = fmaf(__uint_as_float(ua.w), __uint_as_float(ub.w), s);
      } else {
        s = fmaf(bf16lo(ua.x), bf16lo(ub.x), s); s = fmaf(bf16hi(ua.x), bf16hi(ub.x), s);
        s = fmaf(bf16lo(ua.y), bf16lo(ub.y), s); s = fmaf(bf16hi(ua.y), bf16hi(ub.y), s);
        s = fmaf(bf16lo(ua.z), bf16lo(ub.z), s); s = fmaf(bf16hi(ua.z), bf16hi(ub.z), s);
        s = fmaf(bf16lo(ua.w), bf16lo(ub.w), s); s = fmaf(bf16hi(ua.w), bf16hi(ub.w), s);
      }
    }
  } else {
    for (int c = lane; c < n; c += 32) s = fmaf(ldx(a + c), ldx(b + c), s);
  }
  return warp_sum(s);
}

// h[entry, i] = act(x[token] . W_up[e, i, :]); one warp per (entry, i)
template <typename T>
__global__ void __launch_bounds__(256) decode_up_kernel(const T* __restrict__ x, const T* __restrict__ w_up, const int* __restrict__ topk_i,
                                                        T* __restrict__ h, int entries, int k, int H, int I, int expert_offset, int e_local,
                                                        int act) {
  const int lane = threadIdx.x & 31;
  const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (wid >= (long long)entries * I) return;
  const int ent = (int)(wid / I), i = (int)(wid % I);
  const int e = topk_i[ent] - expert_offset;
  if (e < 0 || e >= e_local) return;
  const float v = warp_dot(x + (size_t)(ent / k) * H, w_up + ((size_t)e * I + i) * H, H, lane);
  if (lane == 0) stx(h + (size_t)ent * I + i, act_apply(act, v));
}

// out[token, n] = sum_slot affinity * round(h[entry] . W_down[e, n, :]); one warp per (token, n)
template <typename T>
__global__ void __launch_bounds__(256) decode_down_kernel(const T* __restrict__ h, const T* __restrict__ w_down, const float* __restrict__ topk_w,
                                                          const int* __restrict__ topk_i, T* __restrict__ out, int N, int k, int H, int I,
                                                          int expert_offset, int e_local) {
  const int lane = threadIdx.x & 31;
  const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (wid >= (long long)N * H) return;
  const int tok = (int)(wid / H), n = (int)(wid % H);
  float f = 0.f;
  for (int s = 0; s < k; ++s) {
    const int ent = tok * k + s, e = topk_i[ent] - expert_offset;
    if (e < 0 || e >= e_local) continue;
    float v = warp_dot(h + (size_t)ent * I, w_down + ((size_t)e * H + n) * I, I, lane);
    if constexpr (!std::is_same<T, float>::value) v = __bfloat162float(__float2bfloat16_rn(v));     // the expert's output in the activation type
    f += topk_w[ent] * v;
  }
  if (lane == 0) stx(out + (size_t)tok * H + n, f);
}

// ---- fp32 router: logits, sigmoid scores, the k largest, renormalised ----------------------------------------------------------------
// Block = RT tokens whose rows sit in shared memory as fp32; warp w forms the logits of experts w, w + 8, ... for all RT tokens from ONE
// pass over the expert's weight row, so the router matrix is read once per RT tokens.  Then warp t picks token t's k largest logits
// (largest first, lowest index on ties; the sigmoid is monotonic, so these are the k largest scores) and divides their scores by
// their sum + eps when eps >= 0.
constexpr int RT = 8;
template <typename T>
__global__ void __launch_bounds__(256) router_sigmoid_topk_kernel(const T* __restrict__ x, const float* __restrict__ w, float* __restrict__ logits,
                                                                  float* __restrict__ topk_w, int* __restrict__ topk_i, int N, int W, int E, int k,
                                                                  float renorm_eps) {
  extern __shared__ float rsm[];               // [RT][W] rows, then [RT][E] logits
  float* xs = rsm;
  float* zs = rsm + (size_t)RT * W;
  const int t0 = blockIdx.x * RT, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < RT * W; i += 256) {
    const int t = i / W, c = i % W;
    xs[i] = t0 + t < N ? ldx(x + (size_t)(t0 + t) * W + c) : 0.f;
  }
  __syncthreads();
  for (int e = warp; e < E; e += 8) {
    const float* wr = w + (size_t)e * W;
    float acc[RT];
#pragma unroll
    for (int t = 0; t < RT; ++t) acc[t] = 0.f;
    for (int c = lane; c < W; c += 32) {
      const float wv = __ldg(wr + c);
#pragma unroll
      for (int t = 0; t < RT; ++t) acc[t] = fmaf(xs[t * W + c], wv, acc[t]);
    }
#pragma unroll
    for (int t = 0; t < RT; ++t) {
      const float v = warp_sum(acc[t]);
      if (lane == 0) zs[t * E + e] = v;
    }
  }
  __syncthreads();
  const int t = warp;                          // 8 warps, RT = 8 tokens
  if (t0 + t >= N) return;
  float* z = zs + t * E;
  if (logits)
    for (int e = lane; e < E; e += 32) logits[(size_t)(t0 + t) * E + e] = z[e];
  float sum = 0.f;
  for (int j = 0; j < k; ++j) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = z[e];
      if (v > best || (v == best && e < bi)) { best = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    const float sc = 1.f / (1.f + expf(-best));
    sum += sc;
    if (lane == 0) {
      topk_w[(size_t)(t0 + t) * k + j] = sc;
      topk_i[(size_t)(t0 + t) * k + j] = bi;
      z[bi] = -INFINITY;                       // taken
    }
    __syncwarp();
  }
  if (renorm_eps >= 0.f) {
    const float inv = 1.f / (sum + renorm_eps);
    for (int j = lane; j < k; j += 32) topk_w[(size_t)(t0 + t) * k + j] *= inv;
  }
}

}  // namespace

size_t router_smem_bytes(int W, int E) { return sizeof(float) * (size_t)RT * (size_t)(W + E); }

void router_sigmoid_topk_launch(const void* x, const float* w, float* logits, float* topk_w, int* topk_i, int N, int W, int E, int k,
                                float renorm_eps, bool lp, cudaStream_t st) {
  if (N <= 0) return;
  if (k > E) throw std::runtime_error("router: more experts chosen than there are");
  const size_t smem = router_smem_bytes(W, E);
  if (smem > 200 * 1024) throw std::runtime_error("router: row too wide for the shared-memory kernel");
  const unsigned grid = (unsigned)((N + RT - 1) / RT);
  if (lp) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(router_sigmoid_topk_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    router_sigmoid_topk_kernel<__nv_bfloat16><<<grid, 256, smem, st>>>((const __nv_bfloat16*)x, w, logits, topk_w, topk_i, N, W, E, k, renorm_eps);
  } else {
    if (smem > 48 * 1024) cudaFuncSetAttribute(router_sigmoid_topk_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    router_sigmoid_topk_kernel<float><<<grid, 256, smem, st>>>((const float*)x, w, logits, topk_w, topk_i, N, W, E, k, renorm_eps);
  }
}

void moe_plain_gather_launch(const void* x, const int* row_entry, const int* tile_expert, void* xp, int R, int H, int k, bool lp, cudaStream_t st) {
  if (R <= 0) return;
  if (lp) gather_kernel<__nv_bfloat16><<<R, 128, 0, st>>>((const __nv_bfloat16*)x, row_entry, tile_expert, (__nv_bfloat16*)xp, H, k);
  else gather_kernel<float><<<R, 128, 0, st>>>((const float*)x, row_entry, tile_expert, (float*)xp, H, k);
}

void moe_plain_gemm_launch(const void* a, const void* w, void* c, int R, int N, int K, int act, const int* tile_expert, bool lp, cudaStream_t st) {
  if (R <= 0 || N <= 0) return;
  if (R % 128 != 0) throw std::runtime_error("moe_plain_gemm: the row bound must be a multiple of 128");
  if (R / PT > 65535) throw std::runtime_error("moe_plain_gemm: too many row tiles");
  dim3 grid((N + PT - 1) / PT, R / PT);
  if (lp) grouped_gemm_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)w, (__nv_bfloat16*)c, N, K, act, tile_expert);
  else grouped_gemm_kernel<float><<<grid, 256, 0, st>>>((const float*)a, (const float*)w, (float*)c, N, K, act, tile_expert);
}

void moe_plain_combine_launch(const void* y, const float* topk_w, const int* pos, void* out, int N, int H, int k, bool lp, cudaStream_t st) {
  if (N <= 0) return;
  if (k > 64) throw std::runtime_error("moe_plain_combine: top-k > 64");
  if (lp) combine_kernel<__nv_bfloat16><<<N, 128, 0, st>>>((const __nv_bfloat16*)y, topk_w, pos, (__nv_bfloat16*)out, H, k);
  else combine_kernel<float><<<N, 128, 0, st>>>((const float*)y, topk_w, pos, (float*)out, H, k);
}

void moe_plain_decode_launch(const void* x, const void* w_up, const void* w_down, const float* topk_w, const int* topk_i, void* h, void* out,
                             int N, int k, int H, int I, int expert_offset, int e_local, int act, bool lp, cudaStream_t st) {
  if (N <= 0) return;
  const long long w1 = (long long)N * k * I, w2 = (long long)N * H;
  const unsigned g1 = (unsigned)((w1 + 7) / 8), g2 = (unsigned)((w2 + 7) / 8);
  if (lp) {
    decode_up_kernel<__nv_bfloat16><<<g1, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w_up, topk_i, (__nv_bfloat16*)h, N * k, k, H, I,
                                                        expert_offset, e_local, act);
    decode_down_kernel<__nv_bfloat16><<<g2, 256, 0, st>>>((const __nv_bfloat16*)h, (const __nv_bfloat16*)w_down, topk_w, topk_i, (__nv_bfloat16*)out, N, k,
                                                          H, I, expert_offset, e_local);
  } else {
    decode_up_kernel<float><<<g1, 256, 0, st>>>((const float*)x, (const float*)w_up, topk_i, (float*)h, N * k, k, H, I, expert_offset, e_local, act);
    decode_down_kernel<float><<<g2, 256, 0, st>>>((const float*)h, (const float*)w_down, topk_w, topk_i, (float*)out, N, k, H, I, expert_offset,
                                                  e_local);
  }
}

}  // namespace nxdi
