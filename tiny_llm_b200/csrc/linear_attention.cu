// Linear attention with a matrix state per head, carried from step to step in 32-bit:
//   S_t = diag(a_t) S_(t-1) + (ks k_t) v_t^T,   o_t = S_t^T (qs q_t)        S: [key size, value size]
// The decay a_t is either one constant per head (retention) or one number per key channel and token,
//   a = sigmoid(z + b)^(1/tau) = exp(-softplus(-(z + b)) / tau)             (gated linear attention)
// with z the 32-bit rows of a projection.  Decays, the recurrence and the state are 32-bit; q, k, v are projection
// outputs of the engine's dtype.  The state of a request lives in state[slot, head, key, value] and is read at the
// start of the request's tokens in the step and written back after the last one.
//
// scan: a CTA owns 32 value columns of one (request, head); a thread owns 16 state rows of one column in registers.
// Eight tokens at a time are staged in shared memory (scaled queries and keys, decays); every thread walks them,
// leaves its partial dot products, and the partials of a column are added over the row slices in a fixed order.
// The operations on a state element are those of the sequence, whatever the cut into steps: the same bits.
//
// SEGMENTED (long portions): the tokens of a request are cut into segments; a first kernel walks every segment from
// a zero state and keeps its end state and the product of its decays per row (S_end = diag(A) S_in + B); a second
// finds each segment's S_in from the carried state and the summaries before it and walks the segment again, now
// writing outputs.  The recurrence is linear in S, so the two ways differ by rounding only.
//
// head_norm_gate: y = o / sqrt(mean(o^2) + eps) * w * silu(g) per (token, head), 32-bit in, engine dtype out.
#include "common.cuh"

TLLM_DEFINE_LAST_ERROR

namespace tllm {

constexpr int LA_ROWS = 16;   // state rows per thread
constexpr int LA_COLS = 32;   // value columns per CTA
constexpr int LA_TOK = 8;     // tokens staged at once

__device__ __forceinline__ float gate_decay(float x, float inv_tau) {
  // sigmoid(x)^(1/tau) without forming the sigmoid: exp(-softplus(-x) / tau)
  const float sp = fmaxf(-x, 0.f) + log1pf(expf(-fabsf(x)));
  return expf(-sp * inv_tau);
}

struct ScanArgs {
  const void *q, *k, *v;
  int ldq, ldk, ldv;
  const float* head_decay;   // [heads] or null
  const float* gate;         // [T, heads * kd] rows of ldg values, or null
  int ldg;
  const float* gate_bias;    // [heads * kd]
  float inv_tau, q_scale, k_scale;
  float* state;              // [slots, heads, kd, vd]
  const int* slots;
  const int* cu_q;
  float* out;                // [T, heads * vd]
  int heads, kd, vd;
  // segments: 0 = serial
  int seg, max_segs;
  float* summary;            // [requests, max_segs, heads, (kd * vd) + kd]
  float* carry;              // [requests, heads, kd, vd]
};

// mode 0: serial over the request's tokens, from and to `state`.
// mode 1: a segment from a zero state; writes the end state and the decay products to `summary` (no outputs).
// mode 2: a segment from the state composed of carry and the summaries before it; writes outputs, and the last
//         segment of a request the state.
template <typename T, int MODE>
__global__ void __launch_bounds__(512) linear_attention_scan_kernel(ScanArgs a) {
  extern __shared__ float sm[];
  pdl_trigger();
  const int lane = threadIdx.x, sl = threadIdx.y, nsl = blockDim.y;
  const int kdp = nsl * LA_ROWS;
  float* sq = sm;                       // [LA_TOK][kdp]
  float* sk = sq + LA_TOK * kdp;        // [LA_TOK][kdp]
  float* sa = sk + LA_TOK * kdp;        // [LA_TOK][kdp]
  float* part = sa + LA_TOK * kdp;      // [LA_TOK][nsl][LA_COLS]
  const int h = blockIdx.y;
  const int r = MODE == 0 ? blockIdx.z : blockIdx.z / a.max_segs;
  const int sg = MODE == 0 ? 0 : blockIdx.z % a.max_segs;
  const int col = blockIdx.x * LA_COLS + lane;
  const bool col_ok = col < a.vd;
  const int tid = sl * LA_COLS + lane, nthreads = nsl * LA_COLS;
  const float hd = a.head_decay ? a.head_decay[h] : 1.f;
  pdl_wait();
  int t0 = a.cu_q[r], t1 = a.cu_q[r + 1];
  if (MODE != 0) {
    t0 += sg * a.seg;
    t1 = min(t1, t0 + a.seg);
    if (t0 >= t1) return;
  }
  const bool last = t1 == a.cu_q[r + 1];
  if (MODE == 1 && last) return;   // the last segment's summary is never read
  const T* q = (const T*)a.q;
  const T* k = (const T*)a.k;
  const T* v = (const T*)a.v;
  float* st = a.state + (((size_t)a.slots[r] * a.heads + h) * a.kd) * a.vd;
  float s[LA_ROWS];
  float dprod[LA_ROWS];
#pragma unroll
  for (int i = 0; i < LA_ROWS; ++i) {
    const int row = sl * LA_ROWS + i;
    const bool ok = col_ok && row < a.kd;
    dprod[i] = 1.f;
    if (MODE == 0) {
      s[i] = ok ? st[(size_t)row * a.vd + col] : 0.f;
    } else if (MODE == 1) {
      s[i] = 0.f;
    } else {
      // the state at the segment's start: the carried state walked through the summaries before this segment
      const float* cr = a.carry + (((size_t)r * a.heads + h) * a.kd) * a.vd;
      float x = ok ? cr[(size_t)row * a.vd + col] : 0.f;
      const size_t per = (size_t)a.kd * a.vd + a.kd;
      for (int g = 0; g < sg; ++g) {
        const float* su = a.summary + (((size_t)r * a.max_segs + g) * a.heads + h) * per;
        if (ok) x = fmaf(su[(size_t)a.kd * a.vd + row], x, su[(size_t)row * a.vd + col]);
      }
      s[i] = x;
    }
  }
  for (int tb = t0; tb < t1; tb += LA_TOK) {
    const int nt = min(LA_TOK, t1 - tb);
    for (int idx = tid; idx < LA_TOK * kdp; idx += nthreads) {
      const int tt = idx / kdp, row = idx % kdp;
      float qv = 0.f, kv = 0.f, av = 1.f;
      if (tt < nt && row < a.kd) {
        const size_t t = (size_t)(tb + tt);
        qv = to_f32(q[t * a.ldq + h * a.kd + row]) * a.q_scale;
        kv = to_f32(k[t * a.ldk + h * a.kd + row]) * a.k_scale;
        av = a.gate ? gate_decay(a.gate[t * a.ldg + h * a.kd + row] + a.gate_bias[h * a.kd + row], a.inv_tau) : hd;
      }
      sq[idx] = qv;
      sk[idx] = kv;
      sa[idx] = av;
    }
    float vv[LA_TOK];
#pragma unroll
    for (int tt = 0; tt < LA_TOK; ++tt)
      vv[tt] = (tt < nt && col_ok) ? to_f32(v[(size_t)(tb + tt) * a.ldv + h * a.vd + col]) : 0.f;
    __syncthreads();
#pragma unroll
    for (int tt = 0; tt < LA_TOK; ++tt) {
      if (tt < nt) {
        const float* pq = sq + tt * kdp + sl * LA_ROWS;
        const float* pk = sk + tt * kdp + sl * LA_ROWS;
        const float* pa = sa + tt * kdp + sl * LA_ROWS;
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < LA_ROWS; ++i) {
          s[i] = fmaf(pa[i], s[i], pk[i] * vv[tt]);
          if (MODE == 1) dprod[i] *= pa[i];
          acc = fmaf(s[i], pq[i], acc);
        }
        if (MODE != 1) part[(tt * nsl + sl) * LA_COLS + lane] = acc;
      }
    }
    __syncthreads();
    if (MODE != 1) {
      for (int idx = tid; idx < nt * LA_COLS; idx += nthreads) {
        const int tt = idx / LA_COLS, c = idx % LA_COLS;
        const int oc = blockIdx.x * LA_COLS + c;
        if (oc < a.vd) {
          float o = 0.f;
          for (int x = 0; x < nsl; ++x) o += part[(tt * nsl + x) * LA_COLS + c];
          a.out[(size_t)(tb + tt) * a.heads * a.vd + h * a.vd + oc] = o;
        }
      }
    }
  }
  if (MODE == 1) {
    const size_t per = (size_t)a.kd * a.vd + a.kd;
    float* su = a.summary + (((size_t)r * a.max_segs + sg) * a.heads + h) * per;
#pragma unroll
    for (int i = 0; i < LA_ROWS; ++i) {
      const int row = sl * LA_ROWS + i;
      if (col_ok && row < a.kd) {
        su[(size_t)row * a.vd + col] = s[i];
        if (col == 0) su[(size_t)a.kd * a.vd + row] = dprod[i];
      }
    }
  } else if (MODE == 0 || last) {
#pragma unroll
    for (int i = 0; i < LA_ROWS; ++i) {
      const int row = sl * LA_ROWS + i;
      if (col_ok && row < a.kd) st[(size_t)row * a.vd + col] = s[i];
    }
  }
}

// The state as earlier steps left it, set aside before the segments run: the last segment of a request overwrites the
// state while other segments of the same request may not have read it yet.
__global__ void linear_attention_carry_kernel(const float* __restrict__ state, const int* __restrict__ slots,
                                              float* __restrict__ carry, long long per_request) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.y;
  const float* src = state + (size_t)slots[r] * per_request;
  float* dst = carry + (size_t)r * per_request;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < per_request; i += (long long)gridDim.x * blockDim.x)
    dst[i] = src[i];
}

template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, const T* __restrict__ g,
                                      int ldg, int heads, int vd, float eps, T* __restrict__ out, long long n_rows) {
  pdl_trigger();
  pdl_wait();
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const int lane = threadIdx.x & 31;
  const long long t = row / heads;
  const int h = (int)(row % heads);
  const float* x = o + row * vd;
  float ss = 0.f;
  for (int j = lane; j < vd; j += 32) ss = fmaf(x[j], x[j], ss);
  ss = warp_sum(ss);
  const float r = 1.f / sqrtf(ss / (float)vd + eps);
  const T* gr = g + t * ldg + (size_t)h * vd;
  T* y = out + row * vd;
  for (int j = lane; j < vd; j += 32) {
    const float gv = to_f32(gr[j]);
    const float sg = gv / (1.f + expf(-gv));
    float val = x[j] * r;
    if (w) val *= w[j];
    y[j] = from_f32<T>(val * sg);
  }
}

}  // namespace tllm

using namespace tllm;

// q, k: [T, heads * kd] rows of ldq / ldk values; v: [T, heads * vd] rows of ldv values (dtype: 0 float32, 1 bfloat16).
// Exactly one of head_decay (float32 [heads]) and gate (float32 [T, heads * kd] rows of ldg values, with gate_bias
// [heads * kd] and inv_tau) is given.  out: float32 [T, heads * vd].  seg > 0: segments of that many tokens with
// `summary` (float32, n_requests * max_segs * heads * (kd * vd + kd) values, then n_requests * heads * kd * vd
// values of carry); seg = 0: serial.
extern "C" int tllm_linear_attention_scan(const void* q, const void* k, const void* v, int ldq, int ldk, int ldv,
                                          const float* head_decay, const float* gate, int ldg, const float* gate_bias,
                                          float inv_tau, float q_scale, float k_scale, float* state, const int* slots,
                                          const int* cu_q, float* out, int heads, int kd, int vd, int n_requests,
                                          int max_q_len, int seg, float* summary, int dtype, void* stream) {
  TLLM_REQUIRE(heads > 0 && kd > 0 && vd > 0 && n_requests > 0 && max_q_len > 0, "linear_attention_scan: empty input");
  TLLM_REQUIRE(kd <= 256, "linear_attention_scan: key size %d (at most 256)", kd);
  TLLM_REQUIRE((head_decay != nullptr) != (gate != nullptr), "linear_attention_scan: one of a decay per head and a gate");
  TLLM_REQUIRE(!gate || gate_bias, "linear_attention_scan: a gate needs its bias");
  TLLM_REQUIRE(dtype == TLLM_F32 || dtype == TLLM_BF16, "linear_attention_scan: unknown dtype code %d", dtype);
  TLLM_REQUIRE(heads <= 65535, "linear_attention_scan: %d heads exceed the grid", heads);
  ScanArgs a;
  a.q = q; a.k = k; a.v = v; a.ldq = ldq; a.ldk = ldk; a.ldv = ldv;
  a.head_decay = head_decay; a.gate = gate; a.ldg = ldg; a.gate_bias = gate_bias;
  a.inv_tau = inv_tau; a.q_scale = q_scale; a.k_scale = k_scale;
  a.state = state; a.slots = slots; a.cu_q = cu_q; a.out = out; a.heads = heads; a.kd = kd; a.vd = vd;
  a.seg = 0; a.max_segs = 1; a.summary = nullptr; a.carry = nullptr;
  const int nsl = (kd + LA_ROWS - 1) / LA_ROWS;
  const dim3 block(LA_COLS, nsl);
  const size_t smem = (size_t)(3 * LA_TOK * nsl * LA_ROWS + LA_TOK * nsl * LA_COLS) * sizeof(float);
  const unsigned bx = (unsigned)((vd + LA_COLS - 1) / LA_COLS);
  cudaStream_t s = (cudaStream_t)stream;
  if (seg <= 0 || max_q_len <= seg) {
    TLLM_REQUIRE(n_requests <= 65535, "linear_attention_scan: %d requests exceed the grid", n_requests);
    const dim3 grid(bx, (unsigned)heads, (unsigned)n_requests);
    if (dtype == TLLM_F32)
      TLLM_LAUNCH("linear_attention_scan", (linear_attention_scan_kernel<float, 0>), grid, block, smem, s, a);
    else
      TLLM_LAUNCH("linear_attention_scan", (linear_attention_scan_kernel<__nv_bfloat16, 0>), grid, block, smem, s, a);
    return TLLM_OK;
  }
  TLLM_REQUIRE(summary != nullptr, "linear_attention_scan: segments need a summary buffer");
  a.seg = seg;
  a.max_segs = (max_q_len + seg - 1) / seg;
  TLLM_REQUIRE((long long)a.max_segs * n_requests <= 65535, "linear_attention_scan: %d segments of %d requests exceed the grid", a.max_segs, n_requests);
  const long long per_request = (long long)heads * kd * vd;
  a.summary = summary;
  a.carry = summary + (size_t)n_requests * a.max_segs * heads * ((size_t)kd * vd + kd);
  const dim3 cgrid((unsigned)((per_request + 1023) / 1024 > 64 ? 64 : (per_request + 1023) / 1024), (unsigned)n_requests);
  TLLM_LAUNCH("linear_attention_carry", linear_attention_carry_kernel, cgrid, 256, 0, s, (const float*)state, slots, a.carry, per_request);
  const dim3 grid(bx, (unsigned)heads, (unsigned)(n_requests * a.max_segs));
  if (dtype == TLLM_F32) {
    TLLM_LAUNCH("linear_attention_summary", (linear_attention_scan_kernel<float, 1>), grid, block, smem, s, a);
    TLLM_LAUNCH("linear_attention_segments", (linear_attention_scan_kernel<float, 2>), grid, block, smem, s, a);
  } else {
    TLLM_LAUNCH("linear_attention_summary", (linear_attention_scan_kernel<__nv_bfloat16, 1>), grid, block, smem, s, a);
    TLLM_LAUNCH("linear_attention_segments", (linear_attention_scan_kernel<__nv_bfloat16, 2>), grid, block, smem, s, a);
  }
  return TLLM_OK;
}

// o: float32 [n_rows = T * heads, vd]; w: float32 [vd] or null; g: [T, heads * vd] rows of ldg values; out: [T, heads * vd].
extern "C" int tllm_head_norm_gate(const float* o, const float* w, const void* g, int ldg, int heads, int vd, float eps,
                                   void* out, long long n_rows, int dtype, void* stream) {
  TLLM_REQUIRE(n_rows > 0 && heads > 0 && vd > 0, "head_norm_gate: empty input");
  const int warps = 4;
  const long long blocks = (n_rows + warps - 1) / warps;
  TLLM_REQUIRE(blocks <= 2147483647LL, "head_norm_gate: %lld rows exceed the grid", n_rows);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TLLM_F32)
    TLLM_LAUNCH("head_norm_gate", head_norm_gate_kernel<float>, (unsigned)blocks, warps * 32, 0, s, o, w, (const float*)g, ldg, heads, vd, eps, (float*)out, n_rows);
  else if (dtype == TLLM_BF16)
    TLLM_LAUNCH("head_norm_gate", head_norm_gate_kernel<__nv_bfloat16>, (unsigned)blocks, warps * 32, 0, s, o, w, (const __nv_bfloat16*)g, ldg, heads, vd, eps, (__nv_bfloat16*)out, n_rows);
  else
    TLLM_FAIL(TLLM_ERR_ARG, "head_norm_gate: unknown dtype code %d", dtype);
  return TLLM_OK;
}
