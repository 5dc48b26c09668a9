// Mixture of experts: routing on the device and one grouped product for all experts.
//
// moe_route: per token, s_e = sigmoid(z_e); the `top` experts with the largest s_e + correction_e are chosen (ties:
//   the lower index); their weights are s_e * scale.  One warp per token, 32-bit.
// moe_align: the (token, choice) pairs of the step, numbered token * top + choice, are grouped by expert into tiles
//   of `tile` rows: sorted_rows[tile * tile_rows + i] is a pair's number or -1 (padding), tile_expert[tile] the
//   tile's expert or -1 (no such tile).  The host knows only the upper bound of the tile count.
// moe_linear: out[row] = act(W[expert of the row's tile] . in[row / rows_per_input]) for every row named by
//   sorted_rows.  W: [experts, N, K].  Every output element is one chain of fmaf over ascending k, so a row's
//   result does not depend on the tile it landed in.
// moe_combine: resid[t] += sum_c weight[t, c] * y[t * top + c] (+ sigmoid(gate logit) * shared[t]), choices in the
//   order the router found them.
// gelu: the exact (erf) GELU, element by element.
#include "common.cuh"

TLLM_DEFINE_LAST_ERROR

namespace tllm {

__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752440f)); }

constexpr int ROUTE_PER_LANE = 16;   // experts per lane: at most 512 experts

__global__ void moe_route_kernel(const float* __restrict__ logits, int ld, int n_experts, const float* __restrict__ correction,
                                 float scale, int top, int* __restrict__ ids, float* __restrict__ weights, int n_tokens) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= n_tokens) return;
  const int lane = threadIdx.x & 31;
  float s[ROUTE_PER_LANE], c[ROUTE_PER_LANE];
#pragma unroll
  for (int i = 0; i < ROUTE_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    if (e < n_experts) {
      s[i] = 1.f / (1.f + expf(-logits[(size_t)t * ld + e]));
      c[i] = s[i] + correction[e];
    } else {
      s[i] = 0.f;
      c[i] = -INFINITY;
    }
  }
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    float bs = 0.f;
#pragma unroll
    for (int i = 0; i < ROUTE_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e < n_experts && (c[i] > best)) { best = c[i]; bi = e; bs = s[i]; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      const float os = __shfl_xor_sync(0xffffffffu, bs, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; bs = os; }
    }
    if (lane == 0) {
      ids[(size_t)t * top + k] = bi;
      weights[(size_t)t * top + k] = bs * scale;
    }
#pragma unroll
    for (int i = 0; i < ROUTE_PER_LANE; ++i)
      if (lane + 32 * i == bi) c[i] = -INFINITY;
  }
}

// One CTA.  Shared: counts[n_experts], start[n_experts] (ints).
__global__ void moe_align_kernel(const int* __restrict__ ids, int n_pairs, int n_experts, int tile, int max_tiles,
                                 int* __restrict__ sorted_rows, int* __restrict__ tile_expert) {
  extern __shared__ int sh[];
  int* counts = sh;
  int* start = sh + n_experts;
  pdl_trigger();
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) counts[e] = 0;
  pdl_wait();
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) atomicAdd(&counts[ids[i]], 1);
  for (int i = threadIdx.x; i < max_tiles * tile; i += blockDim.x) sorted_rows[i] = -1;
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < n_experts; ++e) {
      start[e] = at * tile;
      const int nt = (counts[e] + tile - 1) / tile;
      for (int x = 0; x < nt; ++x) tile_expert[at + x] = e;
      at += nt;
      counts[e] = 0;
    }
    for (; at < max_tiles; ++at) tile_expert[at] = -1;
  }
  __syncthreads();
  // Pairs of one expert keep their order (by token, then choice) only up to the order of these atomics; a row's result
  // does not depend on where in its expert's tiles it lies.
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int e = ids[i];
    sorted_rows[start[e] + atomicAdd(&counts[e], 1)] = i;
  }
}

// Tile of TM rows x 64 columns, k in slices of 16; 256 threads, each TM/16 rows x 4 columns.
template <typename T, typename TO, int TM, bool GELU>
__global__ void __launch_bounds__(256) moe_linear_kernel(const T* __restrict__ in, int ld_in, const T* __restrict__ w,
                                                         const int* __restrict__ sorted_rows,
                                                         const int* __restrict__ tile_expert, TO* __restrict__ out,
                                                         int n, int k, int rows_per_input) {
  constexpr int TN = 64, TK = 16, RM = TM / 16;
  __shared__ float sa[TK][TM + 1];
  __shared__ float sb[TK][TN + 1];
  __shared__ int srow[TM];
  pdl_trigger();
  pdl_wait();
  const int e = tile_expert[blockIdx.x];
  if (e < 0) return;
  const int n0 = blockIdx.y * TN;
  const int tid = threadIdx.x;
  if (tid < TM) srow[tid] = sorted_rows[(size_t)blockIdx.x * TM + tid];
  __syncthreads();
  const T* we = w + (size_t)e * n * k;
  const int tr = tid / 16, tc = tid % 16;   // rows tr * RM .., columns tc * 4 ..
  float acc[RM][4];
#pragma unroll
  for (int i = 0; i < RM; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < k; k0 += TK) {
    for (int idx = tid; idx < TM * TK; idx += 256) {
      const int m = idx / TK, kk = idx % TK;
      const int row = srow[m];
      sa[kk][m] = (row >= 0 && k0 + kk < k) ? to_f32(in[(size_t)(row / rows_per_input) * ld_in + k0 + kk]) : 0.f;
    }
    for (int idx = tid; idx < TN * TK; idx += 256) {
      const int c = idx / TK, kk = idx % TK;
      sb[kk][c] = (n0 + c < n && k0 + kk < k) ? to_f32(we[(size_t)(n0 + c) * k + k0 + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float av[RM], bv[4];
#pragma unroll
      for (int i = 0; i < RM; ++i) av[i] = sa[kk][tr * RM + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = sb[kk][tc * 4 + j];
#pragma unroll
      for (int i = 0; i < RM; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < RM; ++i) {
    const int row = srow[tr * RM + i];
    if (row < 0) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = n0 + tc * 4 + j;
      if (c < n) out[(size_t)row * n + c] = from_f32<TO>(GELU ? gelu_erf(acc[i][j]) : acc[i][j]);
    }
  }
}

__global__ void moe_combine_kernel(const float* __restrict__ y, const float* __restrict__ weights, int top,
                                   const float* __restrict__ shared, const float* __restrict__ logits, int ld_logits,
                                   int gate_col, float* __restrict__ resid, int width) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  float g = 0.f;
  if (shared) g = 1.f / (1.f + expf(-logits[(size_t)t * ld_logits + gate_col]));
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float acc = 0.f;
    for (int x = 0; x < top; ++x) acc = fmaf(weights[(size_t)t * top + x], y[((size_t)t * top + x) * width + c], acc);
    if (shared) acc = fmaf(g, shared[(size_t)t * width + c], acc);
    resid[(size_t)t * width + c] += acc;
  }
}

template <typename T>
__global__ void gelu_kernel(const T* __restrict__ x, T* __restrict__ y, long long n) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    y[i] = from_f32<T>(gelu_erf(to_f32(x[i])));
}

}  // namespace tllm

using namespace tllm;

extern "C" int tllm_moe_route(const float* logits, int ld, int n_experts, const float* correction, float scale, int top,
                              int* ids, float* weights, int n_tokens, void* stream) {
  TLLM_REQUIRE(n_tokens > 0 && n_experts > 0 && top > 0 && top <= n_experts, "moe_route: %d of %d experts for %d tokens", top, n_experts, n_tokens);
  TLLM_REQUIRE(n_experts <= 32 * ROUTE_PER_LANE, "moe_route: %d experts (at most %d)", n_experts, 32 * ROUTE_PER_LANE);
  const int warps = 4;
  TLLM_LAUNCH("moe_route", moe_route_kernel, (unsigned)((n_tokens + warps - 1) / warps), warps * 32, 0, (cudaStream_t)stream,
              logits, ld, n_experts, correction, scale, top, ids, weights, n_tokens);
  return TLLM_OK;
}

extern "C" int tllm_moe_align(const int* ids, int n_pairs, int n_experts, int tile, int max_tiles, int* sorted_rows,
                              int* tile_expert, void* stream) {
  TLLM_REQUIRE(n_pairs > 0 && n_experts > 0 && tile > 0 && max_tiles > 0, "moe_align: empty input");
  TLLM_REQUIRE(n_experts <= 4096, "moe_align: %d experts (at most 4096)", n_experts);
  TLLM_LAUNCH("moe_align", moe_align_kernel, 1, 1024, (size_t)2 * n_experts * sizeof(int), (cudaStream_t)stream, ids, n_pairs,
              n_experts, tile, max_tiles, sorted_rows, tile_expert);
  return TLLM_OK;
}

template <typename T, typename TO>
static int moe_linear_launch(const void* in, int ld_in, const void* w, const int* sorted_rows, const int* tile_expert,
                             void* out, int n, int k, int rows_per_input, int tile, int max_tiles, int gelu, cudaStream_t s) {
  const dim3 grid((unsigned)max_tiles, (unsigned)((n + 63) / 64));
#define TLLM_MOE_CASE(TM, G)                                                                                          \
  TLLM_LAUNCH("moe_linear", (moe_linear_kernel<T, TO, TM, G>), grid, 256, 0, s, (const T*)in, ld_in, (const T*)w,      \
              sorted_rows, tile_expert, (TO*)out, n, k, rows_per_input)
  if (tile == 16) { if (gelu) TLLM_MOE_CASE(16, true); else TLLM_MOE_CASE(16, false); }
  else { if (gelu) TLLM_MOE_CASE(64, true); else TLLM_MOE_CASE(64, false); }
#undef TLLM_MOE_CASE
  return TLLM_OK;
}

// in: [rows, k] rows of ld_in values; w: [experts, n, k]; out: [pairs, n] of out_dtype.
extern "C" int tllm_moe_linear(const void* in, int ld_in, const void* w, const int* sorted_rows, const int* tile_expert,
                               void* out, int n, int k, int rows_per_input, int tile, int max_tiles, int gelu, int dtype,
                               int out_dtype, void* stream) {
  TLLM_REQUIRE(n > 0 && k > 0 && rows_per_input > 0 && max_tiles > 0 && (tile == 16 || tile == 64), "moe_linear: sizes do not fit (tile %d)", tile);
  TLLM_REQUIRE(max_tiles <= 2147483647 && (n + 63) / 64 <= 65535, "moe_linear: the grid is too large");
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TLLM_F32 && out_dtype == TLLM_F32)
    return moe_linear_launch<float, float>(in, ld_in, w, sorted_rows, tile_expert, out, n, k, rows_per_input, tile, max_tiles, gelu, s);
  if (dtype == TLLM_BF16 && out_dtype == TLLM_BF16)
    return moe_linear_launch<__nv_bfloat16, __nv_bfloat16>(in, ld_in, w, sorted_rows, tile_expert, out, n, k, rows_per_input, tile, max_tiles, gelu, s);
  if (dtype == TLLM_BF16 && out_dtype == TLLM_F32)
    return moe_linear_launch<__nv_bfloat16, float>(in, ld_in, w, sorted_rows, tile_expert, out, n, k, rows_per_input, tile, max_tiles, gelu, s);
  TLLM_FAIL(TLLM_ERR_ARG, "moe_linear: dtype codes %d -> %d", dtype, out_dtype);
}

extern "C" int tllm_moe_combine(const float* y, const float* weights, int top, const float* shared, const float* logits,
                                int ld_logits, int gate_col, float* resid, int n_tokens, int width, void* stream) {
  TLLM_REQUIRE(n_tokens > 0 && width > 0 && top > 0, "moe_combine: empty input");
  TLLM_REQUIRE(!shared || logits, "moe_combine: a shared expert needs its gate's logits");
  TLLM_LAUNCH("moe_combine", moe_combine_kernel, (unsigned)n_tokens, width >= 1024 ? 256 : 128, 0, (cudaStream_t)stream, y, weights, top,
              shared, logits, ld_logits, gate_col, resid, width);
  return TLLM_OK;
}

extern "C" int tllm_gelu(const void* x, void* y, long long n, int dtype, void* stream) {
  TLLM_REQUIRE(n > 0, "gelu: empty input");
  const long long blocks = (n + 255) / 256;
  const unsigned grid = (unsigned)(blocks > 148 * 16 ? 148 * 16 : blocks);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TLLM_F32)
    TLLM_LAUNCH("gelu", gelu_kernel<float>, grid, 256, 0, s, (const float*)x, (float*)y, n);
  else if (dtype == TLLM_BF16)
    TLLM_LAUNCH("gelu", gelu_kernel<__nv_bfloat16>, grid, 256, 0, s, (const __nv_bfloat16*)x, (__nv_bfloat16*)y, n);
  else
    TLLM_FAIL(TLLM_ERR_ARG, "gelu: unknown dtype code %d", dtype);
  return TLLM_OK;
}
