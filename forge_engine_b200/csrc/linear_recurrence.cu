// Linear attention with a fixed decay per head, carried in a 32-bit state per request:
//   S_t = decay_h * S_(t-1) + k_t v_t^T          (S: [key dim, value dim])
//   o_t = S_t^T q_t
// with q, k, v = act(projection) taken in 32-bit from the projection's output.
//
// One block per (entry, head, stretch of 32 value columns).  The block's 128 threads are
// 4 key-row groups x 32 columns; a thread keeps the state elements (rows g, g + 4, ...;
// its column) in registers for the whole portion and walks the entry's tokens in order,
// LR_CHUNK tokens at a time (their q, k, v staged in shared memory).  The state is read
// from the request's slot before the first token and written back after the last, so a
// prompt cut into portions, or decoded token by token, runs the same additions in the same
// order as the whole prompt at once.
#include "common.cuh"

#define LR_CHUNK 16
#define LR_GROUPS 4

__device__ __forceinline__ float lr_act(float z, int act) { return act == 0 ? z / (1.f + expf(-z)) : z; }

template <typename TI, int ROWS>
__global__ void __launch_bounds__(LR_GROUPS * 32)
linear_recurrence_kernel(const TI* __restrict__ proj, int ld, int q_off, int k_off, int v_off, int act,
                         float* __restrict__ state, const int* __restrict__ slots, const int* __restrict__ cu_tokens,
                         const float* __restrict__ decay, float* __restrict__ out, int heads, int dk, int dv,
                         int state_rows) {
  extern __shared__ float smem[];
  float* qs = smem;                              // [LR_CHUNK][dk]
  float* ks = qs + LR_CHUNK * dk;                // [LR_CHUNK][dk]
  float* vs = ks + LR_CHUNK * dk;                // [LR_CHUNK][32]
  float* part = vs + LR_CHUNK * 32;              // [LR_CHUNK][LR_GROUPS][32]
  pdl_trigger();
  pdl_wait();
  const int entry = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * 32;
  const int g = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = col0 + lane;
  const bool live = col < dv;
  const int begin = cu_tokens[entry], end = cu_tokens[entry + 1];
  const int slot = slots[entry];
  if (slot < 0 || slot >= state_rows || end <= begin) return;
  const float lam = decay[head];
  float* S = state + ((size_t)slot * heads + head) * dk * dv;
  float s[ROWS];
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    const int row = g + i * LR_GROUPS;
    s[i] = (live && row < dk) ? S[(size_t)row * dv + col] : 0.f;
  }
  for (int t0 = begin; t0 < end; t0 += LR_CHUNK) {
    const int count = min(LR_CHUNK, end - t0);
    __syncthreads();
    for (int i = threadIdx.x; i < count * dk; i += blockDim.x) {
      const int t = i / dk, d = i - t * dk;
      const TI* row = proj + (size_t)(t0 + t) * ld + (size_t)head * dk + d;
      qs[i] = lr_act(to_float(row[q_off]), act);
      ks[i] = lr_act(to_float(row[k_off]), act);
    }
    for (int i = threadIdx.x; i < count * 32; i += blockDim.x) {
      const int t = i >> 5, c = col0 + (i & 31);
      vs[i] = c < dv ? lr_act(to_float(proj[(size_t)(t0 + t) * ld + v_off + (size_t)head * dv + c]), act) : 0.f;
    }
    __syncthreads();
    for (int t = 0; t < count; ++t) {
      const float v = vs[t * 32 + lane];
      const float* kt = ks + t * dk;
      const float* qt = qs + t * dk;
      float o = 0.f;
#pragma unroll
      for (int i = 0; i < ROWS; ++i) {
        const int row = g + i * LR_GROUPS;
        if (row < dk) {
          s[i] = fmaf(lam, s[i], kt[row] * v);
          o = fmaf(s[i], qt[row], o);
        }
      }
      part[(t * LR_GROUPS + g) * 32 + lane] = o;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < count * 32; i += blockDim.x) {
      const int t = i >> 5, c = i & 31;
      if (col0 + c < dv) {
        float o = 0.f;
#pragma unroll
        for (int gg = 0; gg < LR_GROUPS; ++gg) o += part[(t * LR_GROUPS + gg) * 32 + c];
        out[(size_t)(t0 + t) * heads * dv + (size_t)head * dv + col0 + c] = o;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    const int row = g + i * LR_GROUPS;
    if (live && row < dk) S[(size_t)row * dv + col] = s[i];
  }
}

FE_EXPORT int fe_linear_recurrence(const void* proj, int dtype, int ld, int q_off, int k_off, int v_off, int act,
                                   float* state, const int* slots, const int* cu_tokens, const float* decay,
                                   float* out, int entries, int heads, int dk, int dv, int state_rows,
                                   cudaStream_t stream) {
  if (entries <= 0) return 0;
  if (dk < 1 || dv < 1 || dk > 512 || heads > 65535) return FE_ERR_BAD_SHAPE;
  dim3 grid(entries, heads, (dv + 31) / 32);
  if (grid.z > 65535) return FE_ERR_TOO_LARGE;
  const size_t smem = sizeof(float) * ((size_t)2 * LR_CHUNK * dk + LR_CHUNK * 32 + LR_CHUNK * LR_GROUPS * 32);
  const int rows = (dk + LR_GROUPS - 1) / LR_GROUPS;
  int rc = 0;
#define LAUNCH(TI, ROWS)                                                                                             \
  do {                                                                                                               \
    if (smem > 48 * 1024)                                                                                            \
      cudaFuncSetAttribute(linear_recurrence_kernel<TI, ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    rc = fe_launch_dependent(linear_recurrence_kernel<TI, ROWS>, grid, dim3(LR_GROUPS * 32), smem, stream,          \
                             (const TI*)proj, ld, q_off, k_off, v_off, act, state, slots, cu_tokens, decay, out,     \
                             heads, dk, dv, state_rows);                                                             \
  } while (0)
#define PICK(TI)                                  \
  do {                                            \
    if (rows <= 8) LAUNCH(TI, 8);                 \
    else if (rows <= 16) LAUNCH(TI, 16);          \
    else if (rows <= 32) LAUNCH(TI, 32);          \
    else if (rows <= 64) LAUNCH(TI, 64);          \
    else LAUNCH(TI, 128);                         \
  } while (0)
  if (dtype == FE_DTYPE_F32) PICK(float);
  else if (dtype == FE_DTYPE_BF16) PICK(bf16);
  else return FE_ERR_BAD_DTYPE;
#undef PICK
#undef LAUNCH
  return rc ? rc : fe_last_error();
}
