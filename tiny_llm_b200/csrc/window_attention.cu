// Attention without softmax over a sliding window plus pooled blocks of older keys, on paged caches.
//
//   weight(i, key) = sigmoid(cap * tanh(q_i . key * scale / cap) + bias_h)         (no cap: the scaled score itself)
//   o_i = sum over visible keys of weight * value, then turned back by the query's position (rotated values)
// Visible to position i: the tokens j with 0 <= i - j < window, and block b (positions b P .. b P + P - 1) iff
// b P + P - 1 <= i - window.  A block's key and value are the means of its tokens' cached keys and values and lie
// in a second paged cache with one row per block.  Scores, weights, sums and angles are 32-bit.
//
// rope_halves_kv_write: rotates the first rot_dims values of every query and key row (value i with i + rot_dims/2)
//   by position * fk[i]; optionally the value rows over their whole size (value m with m + vd/2) by position * fv[m];
//   queries in place, keys and values into their pages.
// pool_kv_blocks: a token that completes a block writes the block's mean key and mean value.
// window_pool_attention: one warp per (token, query head).  32 keys at a time: every lane scores one key, then the
//   warp adds the 32 weighted value rows, lanes across the value's columns.  Blocks first, then tokens, by ascending
//   position: the order of every sum depends on the position alone, not on the step's cut or the batch.
#include "common.cuh"
#include "window_attention.cuh"

TLLM_DEFINE_LAST_ERROR

namespace tllm {

template <typename T>
__global__ void rope_halves_kv_write_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                            const float* __restrict__ fk, int rot_dims, const float* __restrict__ fv,
                                            int n_tokens, int nq, int nk, int nv, int kd, int vd, int row_stride,
                                            T* __restrict__ kcache, T* __restrict__ vcache,
                                            const int* __restrict__ slot_mapping, int page_size, long long k_page_stride,
                                            long long k_head_stride, long long v_page_stride, long long v_head_stride) {
  __shared__ float ck[256], sk[256], cv[256], sv[256];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  if (t >= n_tokens) return;
  const float pos = (float)positions[t];
  const int half_rot = rot_dims / 2, half_v = vd / 2;
  for (int i = threadIdx.x; i < half_rot; i += blockDim.x) {
    const float ang = __fmul_rn(pos, fk[i]);
    sincosf(ang, &sk[i], &ck[i]);
  }
  if (fv)
    for (int i = threadIdx.x; i < half_v; i += blockDim.x) {
      const float ang = __fmul_rn(pos, fv[i]);
      sincosf(ang, &sv[i], &cv[i]);
    }
  __syncthreads();
  T* row = qkv + (size_t)t * row_stride;
  const int slot = slot_mapping[t];
  const long long page = slot / page_size, off = slot % page_size;
  T* kbase = kcache + page * k_page_stride + off * kd;
  T* vbase = vcache + page * v_page_stride + off * vd;
  // rotated pairs of queries and keys
  for (int idx = threadIdx.x; idx < (nq + nk) * half_rot; idx += blockDim.x) {
    const int h = idx / half_rot, i = idx % half_rot;
    const T* src = row + (size_t)h * kd;
    const float u = to_f32(src[i]), v = to_f32(src[i + half_rot]);
    const float c = ck[i], s = sk[i];
    const float ou = fmaf(u, c, -__fmul_rn(v, s)), ov = fmaf(v, c, __fmul_rn(u, s));
    if (h < nq) {
      row[(size_t)h * kd + i] = from_f32<T>(ou);
      row[(size_t)h * kd + i + half_rot] = from_f32<T>(ov);
    } else if (slot >= 0) {
      T* dst = kbase + (long long)(h - nq) * k_head_stride;
      dst[i] = from_f32<T>(ou);
      dst[i + half_rot] = from_f32<T>(ov);
    }
  }
  if (slot < 0) return;
  // the rest of every key row passes unchanged
  const int rest = kd - rot_dims;
  for (int idx = threadIdx.x; idx < nk * rest; idx += blockDim.x) {
    const int h = idx / rest, i = rot_dims + idx % rest;
    kbase[(long long)h * k_head_stride + i] = row[(size_t)(nq + h) * kd + i];
  }
  const T* vsrc = row + (size_t)(nq + nk) * kd;
  if (fv) {
    for (int idx = threadIdx.x; idx < nv * half_v; idx += blockDim.x) {
      const int h = idx / half_v, m = idx % half_v;
      const float u = to_f32(vsrc[(size_t)h * vd + m]), v = to_f32(vsrc[(size_t)h * vd + m + half_v]);
      const float c = cv[m], s = sv[m];
      T* dst = vbase + (long long)h * v_head_stride;
      dst[m] = from_f32<T>(fmaf(u, c, -__fmul_rn(v, s)));
      dst[m + half_v] = from_f32<T>(fmaf(v, c, __fmul_rn(u, s)));
    }
  } else {
    for (int idx = threadIdx.x; idx < nv * vd; idx += blockDim.x)
      vbase[(long long)(idx / vd) * v_head_stride + idx % vd] = vsrc[idx];
  }
}

template <typename T>
__global__ void pool_kv_blocks_kernel(const T* __restrict__ kcache, const T* __restrict__ vcache,
                                      const int* __restrict__ block_table, int max_blocks, T* __restrict__ pk,
                                      T* __restrict__ pv, const int* __restrict__ pool_slots,
                                      const int* __restrict__ positions, const int* __restrict__ token_request, int pool,
                                      int kd, int vd, int page_size, long long k_page_stride, long long k_head_stride,
                                      long long v_page_stride, long long v_head_stride, long long pk_page_stride,
                                      long long pk_head_stride, long long pv_page_stride, long long pv_head_stride) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const int slot = pool_slots[t];
  if (slot < 0) return;   // this token completes no block
  const int p = positions[t], r = token_request[t];
  const int* table = block_table + (size_t)r * max_blocks;
  const int first = p - pool + 1;
  const float inv = 1.f / (float)pool;
  const long long ppage = slot / page_size, poff = slot % page_size;
  for (int e = threadIdx.x; e < kd + vd; e += blockDim.x) {
    const bool is_k = e < kd;
    const int d = is_k ? e : e - kd;
    const T* base = is_k ? kcache + h * k_head_stride + d : vcache + h * v_head_stride + d;
    const long long page_stride = is_k ? k_page_stride : v_page_stride;
    const int row = is_k ? kd : vd;
    float sum = 0.f;
    // eight loads in flight, added in the order of the positions
    for (int j0 = first; j0 <= p; j0 += 8) {
      long long pg[8];
      float x[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) pg[u] = table[min(j0 + u, p) / page_size];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int j = min(j0 + u, p);
        // a token's page outlives its block's completion; a missing one (never) would read page 0 and count as zero
        x[u] = to_f32(base[(pg[u] < 0 ? 0 : pg[u]) * page_stride + (long long)(j % page_size) * row]);
        if (j0 + u > p || pg[u] < 0) x[u] = 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) sum += x[u];
    }
    if (is_k) pk[ppage * pk_page_stride + h * pk_head_stride + poff * kd + d] = from_f32<T>(sum * inv);
    else pv[ppage * pv_page_stride + h * pv_head_stride + poff * vd + d] = from_f32<T>(sum * inv);
  }
}

constexpr int WA_WARPS = 4;
constexpr int WA_MAX_VD = 512;

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const T* __restrict__ k, int kd) {
  float acc = 0.f;
  for (int d = 0; d < kd; ++d) acc = fmaf(q[d], to_f32(k[d]), acc);
  return acc;
}
template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* __restrict__ q, const __nv_bfloat16* __restrict__ k, int kd) {
  float acc = 0.f;
  if ((kd & 7) == 0 && (reinterpret_cast<uintptr_t>(k) & 15) == 0) {
    for (int d = 0; d < kd; d += 8) {
      const uint4 raw = *reinterpret_cast<const uint4*>(k + d);
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const float2 f = __bfloat1622float2(p[x]);
        acc = fmaf(q[d + 2 * x], f.x, acc);
        acc = fmaf(q[d + 2 * x + 1], f.y, acc);
      }
    }
    return acc;
  }
  for (int d = 0; d < kd; ++d) acc = fmaf(q[d], __bfloat162float(k[d]), acc);
  return acc;
}
template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ q, const float* __restrict__ k, int kd) {
  float acc = 0.f;
  if ((kd & 3) == 0 && (reinterpret_cast<uintptr_t>(k) & 15) == 0) {
    for (int d = 0; d < kd; d += 4) {
      const float4 f = *reinterpret_cast<const float4*>(k + d);
      acc = fmaf(q[d], f.x, acc);
      acc = fmaf(q[d + 1], f.y, acc);
      acc = fmaf(q[d + 2], f.z, acc);
      acc = fmaf(q[d + 3], f.w, acc);
    }
    return acc;
  }
  for (int d = 0; d < kd; ++d) acc = fmaf(q[d], k[d], acc);
  return acc;
}

template <typename T>
__global__ void __launch_bounds__(WA_WARPS * 32) window_pool_attention_kernel(WinArgs a) {
  extern __shared__ float sm[];
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x, h = blockIdx.y * WA_WARPS + warp;
  float* sq = sm + (size_t)warp * (a.kd + a.vd);   // the query, later the head's output
  const float bias = h < a.nh ? a.head_bias[h] : 0.f;
  pdl_wait();
  if (h >= a.nh) return;
  const int i = a.positions[t], r = a.token_request[t];
  const int kvh = h / (a.nh / a.nkv);
  const T* qrow = (const T*)a.qkv + (size_t)t * a.row_stride + (size_t)h * a.kd;
  for (int d = lane; d < a.kd; d += 32) sq[d] = to_f32(qrow[d]);
  __syncwarp();
  constexpr int NACC = WA_MAX_VD / 32;
  float acc[NACC];
#pragma unroll
  for (int c = 0; c < NACC; ++c) acc[c] = 0.f;
  const int lo = a.window > 0 ? max(0, i - a.window + 1) : 0;
  const int nblocks = (a.window > 0 && a.pool > 0 && i - a.window - a.pool + 1 >= 0) ? (i - a.window - a.pool + 1) / a.pool + 1 : 0;
  const int ntok = i - lo + 1;
  const int total = nblocks + ntok;
  const int* table = a.table + (size_t)r * a.max_blocks;
  const int* ptable = a.ptable ? a.ptable + (size_t)r * a.pmax_blocks : nullptr;
  for (int base = 0; base < total; base += 32) {
    const int n = base + lane;
    const T* kp = nullptr;
    const T* vp = nullptr;
    if (n < nblocks) {
      const long long page = ptable[n / a.page_size];
      const int off = n % a.page_size;
      if (page >= 0) {
        kp = (const T*)a.pk + page * a.pk_page_stride + kvh * a.pk_head_stride + (long long)off * a.kd;
        vp = (const T*)a.pv + page * a.pv_page_stride + kvh * a.pv_head_stride + (long long)off * a.vd;
      }
    } else if (n < total) {
      const int j = lo + (n - nblocks);
      const long long page = table[j / a.page_size];
      const int off = j % a.page_size;
      if (page >= 0) {
        kp = (const T*)a.k + page * a.k_page_stride + kvh * a.k_head_stride + (long long)off * a.kd;
        vp = (const T*)a.v + page * a.v_page_stride + kvh * a.v_head_stride + (long long)off * a.vd;
      }
    }
    float w = 0.f;
    if (kp) {
      float s = dot_row<T>(sq, kp, a.kd) * a.scale;
      if (a.cap > 0.f) s = a.cap * tanhf(s / a.cap);
      w = 1.f / (1.f + expf(-(s + bias)));
    }
    const int cnt = min(32, total - base);
    for (int x = 0; x < cnt; ++x) {
      const float wx = __shfl_sync(0xffffffffu, w, x);
      const unsigned long long addr = __shfl_sync(0xffffffffu, (unsigned long long)vp, x);
      const T* vr = (const T*)addr;
      if (!vr) continue;
#pragma unroll
      for (int c = 0; c < NACC; ++c) {
        const int d = lane + 32 * c;
        if (d < a.vd) acc[c] = fmaf(wx, to_f32(vr[d]), acc[c]);
      }
    }
  }
  T* orow = (T*)a.out + (size_t)t * a.nh * a.vd + (size_t)h * a.vd;
  if (!a.fv) {
#pragma unroll
    for (int c = 0; c < NACC; ++c) {
      const int d = lane + 32 * c;
      if (d < a.vd) orow[d] = from_f32<T>(acc[c]);
    }
    return;
  }
  float* so = sq + a.kd;
#pragma unroll
  for (int c = 0; c < NACC; ++c) {
    const int d = lane + 32 * c;
    if (d < a.vd) so[d] = acc[c];
  }
  __syncwarp();
  const int half = a.vd / 2;
  const float pos = (float)i;
  for (int m = lane; m < half; m += 32) {
    float sn, cs;
    sincosf(__fmul_rn(pos, a.fv[m]), &sn, &cs);
    const float u = so[m], v = so[m + half];
    // turned back: the rotation by -position
    orow[m] = from_f32<T>(fmaf(u, cs, __fmul_rn(v, sn)));
    orow[m + half] = from_f32<T>(fmaf(v, cs, -__fmul_rn(u, sn)));
  }
}

}  // namespace tllm

using namespace tllm;

extern "C" int tllm_rope_halves_kv_write(void* qkv, const int* positions, const float* fk, int rot_dims, const float* fv,
                                         int n_tokens, int nq, int nk, int nv, int kd, int vd, int row_stride,
                                         void* kcache, void* vcache, const int* slot_mapping, int page_size,
                                         long long k_page_stride, long long k_head_stride, long long v_page_stride,
                                         long long v_head_stride, int dtype, void* stream) {
  TLLM_REQUIRE(n_tokens > 0 && nq > 0 && nk > 0 && nv > 0 && kd > 0 && vd > 0, "rope_halves_kv_write: empty input");
  TLLM_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= kd && rot_dims <= 512 && (rot_dims == 0 || fk),
               "rope_halves_kv_write: %d rotated values of %d (even, at most the key size and 512, with a frequency table)", rot_dims, kd);
  TLLM_REQUIRE(!fv || (vd % 2 == 0 && vd <= 512), "rope_halves_kv_write: rotated values of size %d (even, at most 512)", vd);
  TLLM_REQUIRE(kcache && vcache && slot_mapping && page_size > 0, "rope_halves_kv_write: needs cache pointers, a slot mapping and a page size");
  const int threads = 256;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TLLM_F32)
    TLLM_LAUNCH("rope_halves_kv_write", rope_halves_kv_write_kernel<float>, n_tokens, threads, 0, s, (float*)qkv, positions, fk, rot_dims, fv, n_tokens, nq, nk, nv, kd, vd, row_stride, (float*)kcache, (float*)vcache, slot_mapping, page_size, k_page_stride, k_head_stride, v_page_stride, v_head_stride);
  else if (dtype == TLLM_BF16)
    TLLM_LAUNCH("rope_halves_kv_write", rope_halves_kv_write_kernel<__nv_bfloat16>, n_tokens, threads, 0, s, (__nv_bfloat16*)qkv, positions, fk, rot_dims, fv, n_tokens, nq, nk, nv, kd, vd, row_stride, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, slot_mapping, page_size, k_page_stride, k_head_stride, v_page_stride, v_head_stride);
  else
    TLLM_FAIL(TLLM_ERR_ARG, "rope_halves_kv_write: unknown dtype code %d", dtype);
  return TLLM_OK;
}

extern "C" int tllm_pool_kv_blocks(const void* kcache, const void* vcache, const int* block_table, int max_blocks, void* pk,
                                   void* pv, const int* pool_slots, const int* positions, const int* token_request,
                                   int n_tokens, int nkv, int pool, int kd, int vd, int page_size, long long k_page_stride,
                                   long long k_head_stride, long long v_page_stride, long long v_head_stride,
                                   long long pk_page_stride, long long pk_head_stride, long long pv_page_stride,
                                   long long pv_head_stride, int dtype, void* stream) {
  TLLM_REQUIRE(n_tokens > 0 && nkv > 0 && pool > 0 && kd > 0 && vd > 0 && page_size > 0 && max_blocks > 0, "pool_kv_blocks: empty input");
  TLLM_REQUIRE(nkv <= 65535, "pool_kv_blocks: %d heads exceed the grid", nkv);
  const dim3 grid((unsigned)n_tokens, (unsigned)nkv);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TLLM_F32)
    TLLM_LAUNCH("pool_kv_blocks", pool_kv_blocks_kernel<float>, grid, 128, 0, s, (const float*)kcache, (const float*)vcache, block_table, max_blocks, (float*)pk, (float*)pv, pool_slots, positions, token_request, pool, kd, vd, page_size, k_page_stride, k_head_stride, v_page_stride, v_head_stride, pk_page_stride, pk_head_stride, pv_page_stride, pv_head_stride);
  else if (dtype == TLLM_BF16)
    TLLM_LAUNCH("pool_kv_blocks", pool_kv_blocks_kernel<__nv_bfloat16>, grid, 128, 0, s, (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache, block_table, max_blocks, (__nv_bfloat16*)pk, (__nv_bfloat16*)pv, pool_slots, positions, token_request, pool, kd, vd, page_size, k_page_stride, k_head_stride, v_page_stride, v_head_stride, pk_page_stride, pk_head_stride, pv_page_stride, pv_head_stride);
  else
    TLLM_FAIL(TLLM_ERR_ARG, "pool_kv_blocks: unknown dtype code %d", dtype);
  return TLLM_OK;
}

extern "C" int tllm_window_pool_attention(const WinArgs* args, int dtype, void* stream) {
  const WinArgs& a = *args;
  TLLM_REQUIRE(a.n_tokens > 0 && a.nh > 0 && a.nkv > 0 && a.nh % a.nkv == 0 && a.kd > 0 && a.vd > 0, "window_pool_attention: sizes do not fit");
  TLLM_REQUIRE(a.vd <= WA_MAX_VD, "window_pool_attention: value size %d (at most %d)", a.vd, WA_MAX_VD);
  TLLM_REQUIRE(a.pool <= 0 || (a.pk && a.pv && a.ptable), "window_pool_attention: pooled blocks need their cache and table");
  TLLM_REQUIRE(!a.fv || a.vd % 2 == 0, "window_pool_attention: rotated values need an even size");
  const dim3 grid((unsigned)a.n_tokens, (unsigned)((a.nh + WA_WARPS - 1) / WA_WARPS));
  const size_t smem = (size_t)WA_WARPS * (a.kd + a.vd) * sizeof(float);
  TLLM_REQUIRE(smem <= 48 * 1024, "window_pool_attention: key size %d + value size %d exceed the shared memory", a.kd, a.vd);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TLLM_F32)
    TLLM_LAUNCH("window_pool_attention", window_pool_attention_kernel<float>, grid, WA_WARPS * 32, smem, s, a);
  else if (dtype == TLLM_BF16)
    TLLM_LAUNCH("window_pool_attention", window_pool_attention_kernel<__nv_bfloat16>, grid, WA_WARPS * 32, smem, s, a);
  else
    TLLM_FAIL(TLLM_ERR_ARG, "window_pool_attention: unknown dtype code %d", dtype);
  return TLLM_OK;
}
