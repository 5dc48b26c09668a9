// Gated linear recurrences over the step's tokens, one state vector per request in 32-bit.
//
// minGRU: the gates read the current token only.  The projection's rows hold [z | u | g] of `width` values each:
//   z_t = sigmoid(z + bz),  c_t = u + bu + 1/2 where u + bu >= 0, sigmoid(u + bu) where it is negative,
//   S_t = (1 - z_t) S_(t-1) + z_t c_t   (element by element),   y_t = S_t * silu(g).
// The state of a request lives in state[slot, width] (float32), is read at the start of the request's tokens in
// this step and written back after the last; a request's tokens are the rows [cu_q[r], cu_q[r+1]).
// Everything but the projection's own values is 32-bit: biases, sigmoids, the recurrence.
//
// Two ways to walk a request's tokens.  SERIAL: one thread per (request, channel) walks them in order, the loads
// of eight tokens in flight at a time; the order of every operation is that of the sequence, so the state after
// token t has the same bits however the sequence was cut into steps.  SEGMENTED (long portions): the tokens are cut
// into segments of SEG; a first kernel composes every segment into (A, B) with S_end = A S_in + B; a second
// kernel finds each segment's S_in by walking the summaries of the segments before it and then walks its own
// tokens.  The recurrence is associative, so the two differ by rounding only.
#include "common.cuh"

TLLM_DEFINE_LAST_ERROR

namespace tllm {

// The sigmoid in 32-bit.  For float32 activations it is the library's exponential and an IEEE division; for bfloat16
// activations (whose inputs carry 8 bits) the hardware's exp2 and reciprocal approximations, 32-bit as well, good to
// about 2^-21: a third of the instructions, and these kernels are bound by them.
template <typename T> __device__ __forceinline__ float sigmoid_f(float v) { return 1.f / (1.f + expf(-v)); }
template <> __device__ __forceinline__ float sigmoid_f<__nv_bfloat16>(float v) { return __frcp_rn(1.f + __expf(-v)); }

struct Gate { float z, c; };
template <typename T>
__device__ __forceinline__ Gate min_gru_gate(float zl, float ul, float bz, float bu) {
  Gate g;
  g.z = sigmoid_f<T>(zl + bz);
  const float u = ul + bu;
  g.c = u >= 0.f ? u + 0.5f : sigmoid_f<T>(u);
  return g;
}
__device__ __forceinline__ float min_gru_step(float s, const Gate& g) {
  return fmaf(g.z, g.c, __fmul_rn(1.f - g.z, s));
}

constexpr int AHEAD = 8;   // tokens whose loads are in flight at once

// Walks rows [t0, t1) of one channel from state s; writes y when Y.
template <typename T, bool Y>
__device__ __forceinline__ float min_gru_walk(const T* __restrict__ zug, int ld, int width, int c, float bz, float bu,
                                              int t0, int t1, float s, T* __restrict__ y) {
  for (int t = t0; t < t1; t += AHEAD) {
    float zl[AHEAD], ul[AHEAD], gl[AHEAD];
#pragma unroll
    for (int i = 0; i < AHEAD; ++i) {
      const bool in = t + i < t1;
      const T* row = zug + (size_t)(in ? t + i : t) * ld;
      zl[i] = to_f32(row[c]);
      ul[i] = to_f32(row[width + c]);
      gl[i] = Y ? to_f32(row[2 * width + c]) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < AHEAD; ++i) {
      if (t + i < t1) {
        s = min_gru_step(s, min_gru_gate<T>(zl[i], ul[i], bz, bu));
        if (Y) y[(size_t)(t + i) * width + c] = from_f32<T>(s * (gl[i] * sigmoid_f<T>(gl[i])));
      }
    }
  }
  return s;
}

template <typename T>
__global__ void min_gru_serial_kernel(const T* __restrict__ zug, int ld, const float* __restrict__ bias_z,
                                      const float* __restrict__ bias_u, float* __restrict__ state,
                                      const int* __restrict__ slots, const int* __restrict__ cu_q,
                                      T* __restrict__ y, int width) {
  pdl_trigger();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int r = blockIdx.y;
  const float bz = c < width ? bias_z[c] : 0.f, bu = c < width ? bias_u[c] : 0.f;
  pdl_wait();
  if (c >= width) return;
  float* st = state + (size_t)slots[r] * width + c;
  *st = min_gru_walk<T, true>(zug, ld, width, c, bz, bu, cu_q[r], cu_q[r + 1], *st, y);
}

// Segment k of request r covers rows [cu_q[r] + k SEG, min(cu_q[r+1], cu_q[r] + (k+1) SEG)).
// summary[(r * max_segs + k) * 2 * width + {0, width} + c] = (A, B) of the segment.
template <typename T>
__global__ void min_gru_summary_kernel(const T* __restrict__ zug, int ld, const float* __restrict__ bias_z,
                                       const float* __restrict__ bias_u, const float* __restrict__ state,
                                       const int* __restrict__ slots, const int* __restrict__ cu_q,
                                       float* __restrict__ summary, float* __restrict__ carry, int width, int seg,
                                       int max_segs) {
  pdl_trigger();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int k = blockIdx.y, r = blockIdx.z;
  const float bz = c < width ? bias_z[c] : 0.f, bu = c < width ? bias_u[c] : 0.f;
  pdl_wait();
  if (c >= width) return;
  // the state as earlier steps left it, set aside: the second kernel's last segment overwrites it while other
  // segments of the same request may not have read it yet
  if (k == 0) carry[(size_t)r * width + c] = state[(size_t)slots[r] * width + c];
  const int t0 = cu_q[r] + k * seg, t1 = min(cu_q[r + 1], t0 + seg);
  if (t0 >= t1 || t1 == cu_q[r + 1]) return;   // the last segment's summary is never read
  float a = 1.f, b = 0.f;
  for (int t = t0; t < t1; t += AHEAD) {
    float zl[AHEAD], ul[AHEAD];
#pragma unroll
    for (int i = 0; i < AHEAD; ++i) {
      const T* row = zug + (size_t)(t + i < t1 ? t + i : t) * ld;
      zl[i] = to_f32(row[c]);
      ul[i] = to_f32(row[width + c]);
    }
#pragma unroll
    for (int i = 0; i < AHEAD; ++i) {
      if (t + i < t1) {
        const Gate g = min_gru_gate<T>(zl[i], ul[i], bz, bu);
        a = __fmul_rn(1.f - g.z, a);
        b = min_gru_step(b, g);
      }
    }
  }
  float* out = summary + ((size_t)r * max_segs + k) * 2 * width;
  out[c] = a;
  out[width + c] = b;
}

template <typename T>
__global__ void min_gru_segment_kernel(const T* __restrict__ zug, int ld, const float* __restrict__ bias_z,
                                       const float* __restrict__ bias_u, float* __restrict__ state,
                                       const int* __restrict__ slots, const int* __restrict__ cu_q,
                                       const float* __restrict__ summary, const float* __restrict__ carry,
                                       T* __restrict__ y, int width, int seg, int max_segs) {
  pdl_trigger();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int k = blockIdx.y, r = blockIdx.z;
  const float bz = c < width ? bias_z[c] : 0.f, bu = c < width ? bias_u[c] : 0.f;
  pdl_wait();
  if (c >= width) return;
  const int t0 = cu_q[r] + k * seg, t1 = min(cu_q[r + 1], t0 + seg);
  if (t0 >= t1) return;
  float s = carry[(size_t)r * width + c];
  const float* sum = summary + (size_t)r * max_segs * 2 * width;
  for (int i = 0; i < k; ++i) s = fmaf(sum[(size_t)i * 2 * width + c], s, sum[(size_t)i * 2 * width + width + c]);
  s = min_gru_walk<T, true>(zug, ld, width, c, bz, bu, t0, t1, s, y);
  if (t1 == cu_q[r + 1]) state[(size_t)slots[r] * width + c] = s;
}

}  // namespace tllm

using namespace tllm;

// zug: [T, >= 3 width] rows of `ld` values (dtype: 0 float32, 1 bfloat16); y: [T, width] of the same type.
// max_q_len: the longest run of tokens of one request in this step.  seg > 0: segments of that many tokens with
// `summary` (float32, n_requests * (2 * ceil(max_q_len / seg) + 1) * width values) between the two kernels; seg = 0: serial.
extern "C" int tllm_min_gru_scan(const void* zug, int ld, const float* bias_z, const float* bias_u, float* state,
                                 const int* slots, const int* cu_q, void* y, int width, int n_requests, int max_q_len,
                                 int seg, float* summary, int dtype, void* stream) {
  TLLM_REQUIRE(width > 0 && n_requests > 0 && max_q_len > 0 && ld >= 3 * width,
               "min_gru_scan: width %d, %d requests, longest run %d, row stride %d", width, n_requests, max_q_len, ld);
  TLLM_REQUIRE(dtype == TLLM_F32 || dtype == TLLM_BF16, "min_gru_scan: unknown dtype code %d", dtype);
  TLLM_REQUIRE(n_requests <= 65535, "min_gru_scan: %d requests exceed the grid", n_requests);
  const int threads = width >= 128 ? 128 : 64;
  const unsigned bx = (unsigned)((width + threads - 1) / threads);
  cudaStream_t s = (cudaStream_t)stream;
  if (seg <= 0 || max_q_len <= seg) {
    const dim3 grid(bx, (unsigned)n_requests);
    if (dtype == TLLM_F32)
      TLLM_LAUNCH("min_gru_scan", min_gru_serial_kernel<float>, grid, threads, 0, s, (const float*)zug, ld, bias_z, bias_u, state, slots, cu_q, (float*)y, width);
    else
      TLLM_LAUNCH("min_gru_scan", min_gru_serial_kernel<__nv_bfloat16>, grid, threads, 0, s, (const __nv_bfloat16*)zug, ld, bias_z, bias_u, state, slots, cu_q, (__nv_bfloat16*)y, width);
    return TLLM_OK;
  }
  TLLM_REQUIRE(summary != nullptr, "min_gru_scan: segments need a summary buffer");
  const int max_segs = (max_q_len + seg - 1) / seg;
  TLLM_REQUIRE(max_segs <= 65535, "min_gru_scan: %d segments exceed the grid", max_segs);
  const dim3 grid(bx, (unsigned)max_segs, (unsigned)n_requests);
  float* carry = summary + (size_t)n_requests * max_segs * 2 * width;
  if (dtype == TLLM_F32) {
    TLLM_LAUNCH("min_gru_summary", min_gru_summary_kernel<float>, grid, threads, 0, s, (const float*)zug, ld, bias_z, bias_u, state, slots, cu_q, summary, carry, width, seg, max_segs);
    TLLM_LAUNCH("min_gru_segment", min_gru_segment_kernel<float>, grid, threads, 0, s, (const float*)zug, ld, bias_z, bias_u, state, slots, cu_q, summary, carry, (float*)y, width, seg, max_segs);
  } else {
    TLLM_LAUNCH("min_gru_summary", min_gru_summary_kernel<__nv_bfloat16>, grid, threads, 0, s, (const __nv_bfloat16*)zug, ld, bias_z, bias_u, state, slots, cu_q, summary, carry, width, seg, max_segs);
    TLLM_LAUNCH("min_gru_segment", min_gru_segment_kernel<__nv_bfloat16>, grid, threads, 0, s, (const __nv_bfloat16*)zug, ld, bias_z, bias_u, state, slots, cu_q, summary, carry, (__nv_bfloat16*)y, width, seg, max_segs);
  }
  return TLLM_OK;
}
