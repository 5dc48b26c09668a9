// Attention without softmax over a sliding window plus pooled blocks of older keys, on the tensor cores
// (bfloat16, mma.sync.m16n8k16), compiled per (key size, value size).  The rule of visibility and the weight
//   sigmoid(cap * tanh(q . k * scale / cap) + bias_h)
// are those of window_attention.cu; scores, weights and sums are 32-bit.
//
// A CTA owns up to 64 rows = (token, query head of the group) of one (request, key/value head): as many whole tokens
// as fit, so the heads of a group share the key and value tiles; four warps of 16 rows.  Keys come in tiles of 32, first the pooled blocks the last
// row can see, then the tokens from the first row's window on; each tile is gathered page by page with 16-byte
// cp.async copies, four threads per row, two tiles in flight.  S = Q K^T with the queries held in registers; the
// weights are formed where the scores lie, and enter the P V product as two bfloat16 terms hi + lo (16 mantissa
// bits), V taken as it lies in the cache through transposing ldmatrix loads.  A head's output is turned back by the
// query's position in the accumulators themselves: column m and column m + VD/2 belong to the same thread.
#include "common.cuh"
#include "window_attention.cuh"

TLLM_DEFINE_LAST_ERROR

#ifndef TLLM_HEAD_DIM
#define TLLM_HEAD_DIM 64
#endif
#ifndef TLLM_VALUE_DIM
#define TLLM_VALUE_DIM 128
#endif

namespace tllm {

constexpr int KD = TLLM_HEAD_DIM, VD = TLLM_VALUE_DIM;
constexpr int BM = 64, BN = 32, NTHREADS = 128;
constexpr int LDK = KD + 8, LDV = VD + 8;
constexpr int NO_KEY = -2147483647 - 1;
static_assert(KD % 16 == 0 && VD % 16 == 0 && KD <= 128 && VD <= 128, "key and value sizes: multiples of 16 up to 128");

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void ldsm4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void ldsm4_t(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float* c, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&v);
}
// a weight as two bfloat16 terms: hi = round(p), lo = round(p - hi)
__device__ __forceinline__ void split2(float p0, float p1, unsigned& hi, unsigned& lo) {
  const __nv_bfloat16 h0 = __float2bfloat16_rn(p0), h1 = __float2bfloat16_rn(p1);
  hi = pack_bf16(__bfloat162float(h0), __bfloat162float(h1));
  lo = pack_bf16(p0 - __bfloat162float(h0), p1 - __bfloat162float(h1));
}

// splits > 1 (few rows, many keys: decoded tokens): blockIdx.x also names one of `splits` runs of the key tiles; every
// run adds its part of the sums into the zeroed float32 buffer `acc` [tokens, heads * VD] (the weights are not
// normalised over the keys, so parts simply add), and window_attention_finish_kernel turns the sums back and stores them.
__global__ void __launch_bounds__(NTHREADS) window_pool_attention_mma_kernel(WinArgs a, const int* __restrict__ cu_q,
                                                                             const int* __restrict__ q_start, int splits,
                                                                             float* __restrict__ acc) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [BM][LDK]
  __nv_bfloat16* sK = sQ + BM * LDK;                                // [2][BN][LDK]
  __nv_bfloat16* sV = sK + 2 * BN * LDK;                            // [2][BN][LDV]
  int* sCode = reinterpret_cast<int*>(sV + 2 * BN * LDV);           // [2][BN]: a token's position, -(a block's end + 1), NO_KEY
  pdl_trigger();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int r = blockIdx.z, g = blockIdx.y;
  const int G = a.nh / a.nkv;
  pdl_wait();
  const int q0 = cu_q[r], qn = cu_q[r + 1] - q0, start = q_start[r];
  const int TPT = BM / G;                      // whole tokens per tile: row m is (token m / G, head m % G), m < TPT * G
  const int tok_lo = (blockIdx.x / splits) * TPT;
  const int split = blockIdx.x % splits;
  if (tok_lo >= qn) return;
  const int tok_hi = min(qn - 1, tok_lo + TPT - 1);
  const int i_min = start + tok_lo, i_max = start + tok_hi;
  const int W = a.window, P = a.pool;
  const int nblk = (W > 0 && P > 0 && i_max - W - P + 1 >= 0) ? (i_max - W - P + 1) / P + 1 : 0;
  const int lo = W > 0 ? max(0, i_min - W + 1) : 0;
  const int total = nblk + (i_max - lo + 1);
  const int all_tiles = (total + BN - 1) / BN;
  const int per_split = (all_tiles + splits - 1) / splits;
  const int kt0 = split * per_split, ntiles = min(all_tiles, kt0 + per_split);   // this CTA's tiles: [kt0, ntiles)
  if (kt0 >= ntiles) return;
  const int* table = a.table + (size_t)r * a.max_blocks;
  const int* ptable = a.ptable ? a.ptable + (size_t)r * a.pmax_blocks : nullptr;
  const __nv_bfloat16* qkv = (const __nv_bfloat16*)a.qkv;

  // the queries of the tile
  for (int idx = tid; idx < BM * (KD / 8); idx += NTHREADS) {
    const int m = idx / (KD / 8), c = (idx % (KD / 8)) * 8;
    const bool ok = m < TPT * G && tok_lo + m / G < qn;
    const __nv_bfloat16* src = qkv + (size_t)(q0 + (ok ? tok_lo + m / G : 0)) * a.row_stride + (size_t)(g * G + (ok ? m % G : 0)) * KD + c;
    cp_async16(sQ + m * LDK + c, src, ok);
  }
  auto load_tile = [&](int kt, int stage) {
    const int n = tid >> 2, part = tid & 3;
    const int idx = kt * BN + n;
    const __nv_bfloat16 *ksrc = qkv, *vsrc = qkv;
    int code = NO_KEY;
    if (idx < nblk) {
      const long long page = ptable[idx / a.page_size];
      const int off = idx % a.page_size;
      if (page >= 0) {
        ksrc = (const __nv_bfloat16*)a.pk + page * a.pk_page_stride + g * a.pk_head_stride + (long long)off * KD;
        vsrc = (const __nv_bfloat16*)a.pv + page * a.pv_page_stride + g * a.pv_head_stride + (long long)off * VD;
        code = -(idx * P + P);
      }
    } else if (idx < total) {
      const int j = lo + idx - nblk;
      const long long page = table[j / a.page_size];
      const int off = j % a.page_size;
      if (page >= 0) {
        ksrc = (const __nv_bfloat16*)a.k + page * a.k_page_stride + g * a.k_head_stride + (long long)off * KD;
        vsrc = (const __nv_bfloat16*)a.v + page * a.v_page_stride + g * a.v_head_stride + (long long)off * VD;
        code = j;
      }
    }
    const bool ok = code != NO_KEY;
    __nv_bfloat16* kd_ = sK + (stage * BN + n) * LDK;
    __nv_bfloat16* vd_ = sV + (stage * BN + n) * LDV;
#pragma unroll
    for (int c = part * 8; c < KD; c += 32) cp_async16(kd_ + c, ksrc + (ok ? c : 0), ok);
#pragma unroll
    for (int c = part * 8; c < VD; c += 32) cp_async16(vd_ + c, vsrc + (ok ? c : 0), ok);
    if (part == 0) sCode[stage * BN + n] = code;
  };
  load_tile(kt0, 0);
  asm volatile("cp.async.commit_group;");

  // this thread's two rows: (token, head), position and bias
  const int rA = warp * 16 + (lane >> 2), rB = rA + 8;
  const bool okA = rA < TPT * G && tok_lo + rA / G < qn, okB = rB < TPT * G && tok_lo + rB / G < qn;
  const int iA = okA ? start + tok_lo + rA / G : -1, iB = okB ? start + tok_lo + rB / G : -1;
  const int hA = g * G + (okA ? rA % G : 0), hB = g * G + (okB ? rB % G : 0);
  const float bA = a.head_bias[hA], bB = a.head_bias[hB];
  const float scale = a.scale, cap = a.cap, inv_cap = a.cap > 0.f ? 1.f / a.cap : 0.f;

  unsigned qf[KD / 16][4];
  float o[VD / 8][4];
#pragma unroll
  for (int x = 0; x < VD / 8; ++x) o[x][0] = o[x][1] = o[x][2] = o[x][3] = 0.f;

  for (int kt = kt0; kt < ntiles; ++kt) {
    const int stage = (kt - kt0) & 1;
    if (kt + 1 < ntiles) load_tile(kt + 1, stage ^ 1);
    asm volatile("cp.async.commit_group;");
    asm volatile("cp.async.wait_group 1;");
    __syncthreads();
    if (kt == kt0) {
#pragma unroll
      for (int kk = 0; kk < KD / 16; ++kk)
        ldsm4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], sQ + (warp * 16 + (lane & 15)) * LDK + kk * 16 + (lane >> 4) * 8);
    }
    float s[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
    const __nv_bfloat16* kbase = sK + stage * BN * LDK;
#pragma unroll
    for (int kk = 0; kk < KD / 16; ++kk) {
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        unsigned b0, b1, b2, b3;
        ldsm4(b0, b1, b2, b3, kbase + (j * 8 + (lane & 7) + (lane >> 4) * 8) * LDK + kk * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(s[j], qf[kk], b0, b1);
        mma_bf16(s[j + 1], qf[kk], b2, b3);
      }
    }
    // weights, in 32-bit, where the scores lie
    unsigned phi[4][2], plo[4][2];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float p[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int code = sCode[stage * BN + j * 8 + (lane & 3) * 2 + (c & 1)];
        const int i = c < 2 ? iA : iB;
        bool vis;
        if (code >= 0) vis = code <= i && (W <= 0 || i - code < W);
        else vis = code != NO_KEY && (-code - 1) <= i - W;
        float x = s[j][c] * scale;
        if (cap > 0.f) x = cap * (1.f - __fdividef(2.f, 1.f + __expf(2.f * x * inv_cap)));   // cap tanh(x / cap)
        x += c < 2 ? bA : bB;
        p[c] = vis ? __fdividef(1.f, 1.f + __expf(-x)) : 0.f;   // the hardware's exp2 and reciprocal, 32-bit, about 2^-21
      }
      split2(p[0], p[1], phi[j][0], plo[j][0]);
      split2(p[2], p[3], phi[j][1], plo[j][1]);
    }
    const __nv_bfloat16* vbase = sV + stage * BN * LDV;
#pragma unroll
    for (int kc = 0; kc < 2; ++kc) {
      const unsigned ah[4] = {phi[2 * kc][0], phi[2 * kc][1], phi[2 * kc + 1][0], phi[2 * kc + 1][1]};
      const unsigned al[4] = {plo[2 * kc][0], plo[2 * kc][1], plo[2 * kc + 1][0], plo[2 * kc + 1][1]};
#pragma unroll
      for (int nv = 0; nv < VD / 8; nv += 2) {
        unsigned b0, b1, b2, b3;
        ldsm4_t(b0, b1, b2, b3, vbase + (kc * 16 + (lane & 15)) * LDV + nv * 8 + (lane >> 4) * 8);
        mma_bf16(o[nv], ah, b0, b1);
        mma_bf16(o[nv], al, b0, b1);
        mma_bf16(o[nv + 1], ah, b2, b3);
        mma_bf16(o[nv + 1], al, b2, b3);
      }
    }
    __syncthreads();
  }
  asm volatile("cp.async.wait_group 0;");

  __nv_bfloat16* out = (__nv_bfloat16*)a.out;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    if (!(half ? okB : okA)) continue;
    const int row = half ? rB : rA, i = half ? iB : iA, h = half ? hB : hA;
    __nv_bfloat16* dst = out + (size_t)(q0 + tok_lo + row / G) * a.nh * VD + (size_t)h * VD;
    if (splits > 1) {
      float* part = acc + (size_t)(q0 + tok_lo + row / G) * a.nh * VD + (size_t)h * VD;
#pragma unroll
      for (int x = 0; x < VD / 8; ++x) {
        const int m = x * 8 + (lane & 3) * 2;
        atomicAdd(part + m, o[x][half * 2]);
        atomicAdd(part + m + 1, o[x][half * 2 + 1]);
      }
      continue;
    }
    if (a.fv) {
      const float pos = (float)i;
#pragma unroll
      for (int x = 0; x < VD / 16; ++x)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int m = x * 8 + (lane & 3) * 2 + c;
          float sn, cs;
          sincosf(__fmul_rn(pos, a.fv[m]), &sn, &cs);
          const float u = o[x][half * 2 + c], v = o[x + VD / 16][half * 2 + c];
          dst[m] = __float2bfloat16_rn(fmaf(u, cs, __fmul_rn(v, sn)));           // turned back: rotation by -position
          dst[m + VD / 2] = __float2bfloat16_rn(fmaf(v, cs, -__fmul_rn(u, sn)));
        }
    } else {
#pragma unroll
      for (int x = 0; x < VD / 8; ++x) {
        const int m = x * 8 + (lane & 3) * 2;
        *reinterpret_cast<unsigned*>(dst + m) = pack_bf16(o[x][half * 2], o[x][half * 2 + 1]);
      }
    }
  }
}

// One warp per (token, head): the sums of the key runs, turned back by the token's position (when values are rotated),
// stored in bfloat16; the buffer is handed back zeroed.
__global__ void window_attention_finish_kernel(float* __restrict__ acc, const int* __restrict__ positions,
                                               const float* __restrict__ fv, __nv_bfloat16* __restrict__ out, int nh,
                                               long long n_rows) {
  pdl_trigger();
  pdl_wait();
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const int lane = threadIdx.x & 31;
  float* src = acc + row * VD;
  __nv_bfloat16* dst = out + row * VD;
  const float pos = (float)positions[row / nh];
  for (int m = lane; m < VD / 2; m += 32) {
    const float u = src[m], v = src[m + VD / 2];
    src[m] = 0.f;
    src[m + VD / 2] = 0.f;
    if (fv) {
      float sn, cs;
      sincosf(__fmul_rn(pos, fv[m]), &sn, &cs);
      dst[m] = __float2bfloat16_rn(fmaf(u, cs, __fmul_rn(v, sn)));
      dst[m + VD / 2] = __float2bfloat16_rn(fmaf(v, cs, -__fmul_rn(u, sn)));
    } else {
      dst[m] = __float2bfloat16_rn(u);
      dst[m + VD / 2] = __float2bfloat16_rn(v);
    }
  }
}

}  // namespace tllm

using namespace tllm;

// splits > 1: the key tiles of every row tile in that many runs, summed through `acc` (float32 [tokens, heads * VD],
// zeroed; handed back zeroed).
extern "C" int tllm_window_pool_attention_mma(const WinArgs* args, const int* cu_q, const int* q_start, int n_requests,
                                              int max_q_len, int splits, float* acc, void* stream) {
  const WinArgs& a = *args;
  TLLM_REQUIRE(a.kd == KD && a.vd == VD, "window_pool_attention_mma: built for keys of %d and values of %d, not %d and %d", KD, VD, a.kd, a.vd);
  TLLM_REQUIRE(a.n_tokens > 0 && n_requests > 0 && max_q_len > 0 && a.nh > 0 && a.nkv > 0 && a.nh % a.nkv == 0, "window_pool_attention_mma: sizes do not fit");
  const int G = a.nh / a.nkv;
  TLLM_REQUIRE(G <= BM, "window_pool_attention_mma: %d heads per key/value head (at most %d)", G, BM);
  TLLM_REQUIRE(a.pool <= 0 || (a.pk && a.pv && a.ptable && a.window > 0), "window_pool_attention_mma: pooled blocks need their cache, their table and a window");
  TLLM_REQUIRE(a.row_stride % 8 == 0 && ((uintptr_t)a.qkv & 15) == 0, "window_pool_attention_mma: query rows must be 16-byte aligned");
  TLLM_REQUIRE(a.nkv <= 65535 && n_requests <= 65535, "window_pool_attention_mma: the grid is too large");
  const size_t smem = (size_t)(BM * LDK + 2 * BN * LDK + 2 * BN * LDV) * sizeof(__nv_bfloat16) + 2 * BN * sizeof(int);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(window_pool_attention_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) TLLM_FAIL(TLLM_ERR_CUDA, "window_pool_attention_mma: %s", cudaGetErrorString(e));
    configured = true;
  }
  const int tokens_per_tile = BM / G;
  TLLM_REQUIRE(splits >= 1 && (splits == 1 || acc != nullptr), "window_pool_attention_mma: key runs need a float32 buffer");
  const dim3 grid((unsigned)((max_q_len + tokens_per_tile - 1) / tokens_per_tile * splits), (unsigned)a.nkv, (unsigned)n_requests);
  TLLM_LAUNCH("window_pool_attention_mma", window_pool_attention_mma_kernel, grid, NTHREADS, smem, (cudaStream_t)stream, a, cu_q, q_start, splits, acc);
  if (splits > 1) {
    const long long n_rows = (long long)a.n_tokens * a.nh;
    TLLM_LAUNCH("window_attention_finish", window_attention_finish_kernel, (unsigned)((n_rows + 3) / 4), 128, 0, (cudaStream_t)stream,
                acc, a.positions, a.fv, (__nv_bfloat16*)a.out, a.nh, n_rows);
  }
  return TLLM_OK;
}
