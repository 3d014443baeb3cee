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

// ---------------------------------------------------------------------------
// The same recurrence for long portions, chunk-parallel.  An entry's tokens are cut into
// chunks of LC (from the entry's first token of this step).  With S the state before a
// chunk and t, j counting inside it,
//   o_t = sum_{j <= t} decay^(t - j) (q_t . k_j) v_j  +  decay^(t + 1) S^T q_t
//   S'  = decay^len S + sum_j decay^(len - 1 - j) k_j v_j^T
// Kernel 1 (a block per chunk and head) takes the first sum and the second line's sum;
// kernel 2 walks an entry's chunks in order, element by element of the state, leaving every
// chunk's incoming state where its sum was; kernel 3 (a block per chunk and head) adds the
// state's share.  All products and sums are 32-bit.
// ---------------------------------------------------------------------------
#define LC 64

// Which entry and which of its chunks a global chunk index is; false past the last one.
__device__ __forceinline__ bool lr_locate(const int* cu_tokens, int entries, int chunk, int* entry, int* local,
                                          int* first_chunk) {
  int seen = 0;
  for (int e = 0; e < entries; ++e) {
    const int n = (cu_tokens[e + 1] - cu_tokens[e] + LC - 1) / LC;
    if (chunk < seen + n) {
      *entry = e;
      *local = chunk - seen;
      *first_chunk = seen;
      return true;
    }
    seen += n;
  }
  return false;
}

// Shared-memory layout of the chunk kernels: q row-major [LC][dk]; k transposed [dk][LCP], so
// that four neighbouring keys are one 16-byte load; v [LC][dv] and the state [dk][dv] with four
// neighbouring columns per load.  A thread owns two rows (32 apart) and four columns of an
// output tile: 8 multiply-adds per three loads.  dv is a multiple of 4.
#define LCP (LC + 4)

__device__ __forceinline__ void fma4(float* acc, float a, const float4& b) {
  acc[0] = fmaf(a, b.x, acc[0]);
  acc[1] = fmaf(a, b.y, acc[1]);
  acc[2] = fmaf(a, b.z, acc[2]);
  acc[3] = fmaf(a, b.w, acc[3]);
}

template <typename TI>
__global__ void __launch_bounds__(256)
lr_chunk_local_kernel(const TI* __restrict__ proj, int ld, int q_off, int k_off, int v_off, int act,
                      const int* __restrict__ cu_tokens, int entries, const float* __restrict__ decay,
                      float* __restrict__ out, float* __restrict__ sums, int heads, int dk, int dv) {
  extern __shared__ __align__(16) float smem[];
  float* qs = smem;                       // [LC][dk]
  float* kt = qs + LC * dk;               // [dk][LCP]
  float* vs = kt + dk * LCP;              // [LC][dv]
  float* as = vs + LC * dv;               // [LC][LCP]
  float* pw = as + LC * LCP;              // [LC + 1] powers of the decay
  pdl_trigger();
  pdl_wait();
  int entry, local, first;
  if (!lr_locate(cu_tokens, entries, blockIdx.x, &entry, &local, &first)) return;
  const int head = blockIdx.y;
  const int t0 = cu_tokens[entry] + local * LC;
  const int len = min(LC, cu_tokens[entry + 1] - t0);
  const float lam = decay[head];
  for (int i = threadIdx.x; i <= LC; i += blockDim.x) pw[i] = powf(lam, (float)i);
#pragma unroll 8
  for (int i = threadIdx.x; i < LC * dk; i += blockDim.x) {
    const int t = i / dk, d = i - t * dk;
    float q = 0.f, k = 0.f;
    if (t < len) {
      const TI* row = proj + (size_t)(t0 + t) * ld + (size_t)head * dk + d;
      q = lr_act(to_float(row[q_off]), act);
      k = lr_act(to_float(row[k_off]), act);
    }
    qs[i] = q;
    kt[d * LCP + t] = k;
  }
#pragma unroll 8
  for (int i = threadIdx.x; i < LC * dv; i += blockDim.x) {
    const int t = i / dv, c = i - t * dv;
    vs[i] = t < len ? lr_act(to_float(proj[(size_t)(t0 + t) * ld + v_off + (size_t)head * dv + c]), act) : 0.f;
  }
  __syncthreads();
  // weights of the chunk's own keys: as[t][j] = decay^(t - j) q_t . k_j for j <= t, else 0
  for (int item = threadIdx.x; item < 32 * (LC / 4); item += blockDim.x) {
    const int tp = item / (LC / 4), j4 = (item - tp * (LC / 4)) * 4;
    const int t1 = tp, t2 = tp + 32;
    float a1[4] = {0.f, 0.f, 0.f, 0.f}, a2[4] = {0.f, 0.f, 0.f, 0.f};
    if (j4 <= t2) {
      const float* q1 = qs + t1 * dk;
      const float* q2 = qs + t2 * dk;
      for (int d = 0; d < dk; ++d) {
        const float4 k4 = *reinterpret_cast<const float4*>(kt + d * LCP + j4);
        fma4(a1, q1[d], k4);
        fma4(a2, q2[d], k4);
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int j = j4 + e;
      as[t1 * LCP + j] = j <= t1 ? a1[e] * pw[t1 - j] : 0.f;
      as[t2 * LCP + j] = j <= t2 ? a2[e] * pw[t2 - j] : 0.f;
    }
  }
  __syncthreads();
  const int dv4 = dv >> 2;
  for (int item = threadIdx.x; item < 32 * dv4; item += blockDim.x) {
    const int tp = item / dv4, c = (item - tp * dv4) * 4;
    const int t1 = tp, t2 = tp + 32;
    float o1[4] = {0.f, 0.f, 0.f, 0.f}, o2[4] = {0.f, 0.f, 0.f, 0.f};
    const int last = min(len, t2 + 1);
    for (int j = 0; j < last; ++j) {
      const float4 v4 = *reinterpret_cast<const float4*>(vs + j * dv + c);
      fma4(o1, as[t1 * LCP + j], v4);
      fma4(o2, as[t2 * LCP + j], v4);
    }
    if (t1 < len) store4(out + (size_t)(t0 + t1) * heads * dv + (size_t)head * dv + c, o1);
    if (t2 < len) store4(out + (size_t)(t0 + t2) * heads * dv + (size_t)head * dv + c, o2);
  }
  // what the chunk adds to the state: sum_j decay^(len - 1 - j) k_j v_j^T
  float* sum = sums + ((size_t)blockIdx.x * heads + head) * dk * dv;
  const int half = (dk + 1) >> 1;
  for (int item = threadIdx.x; item < half * dv4; item += blockDim.x) {
    const int rp = item / dv4, c = (item - rp * dv4) * 4;
    const int r1 = rp, r2 = rp + half;
    const bool second = r2 < dk;
    float s1[4] = {0.f, 0.f, 0.f, 0.f}, s2[4] = {0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < len; ++j) {
      const float4 v4 = *reinterpret_cast<const float4*>(vs + j * dv + c);
      const float w = pw[len - 1 - j];
      fma4(s1, w * kt[r1 * LCP + j], v4);
      if (second) fma4(s2, w * kt[r2 * LCP + j], v4);
    }
    store4(sum + (size_t)r1 * dv + c, s1);
    if (second) store4(sum + (size_t)r2 * dv + c, s2);
  }
}

__global__ void lr_chunk_scan_kernel(float* __restrict__ state, const int* __restrict__ slots,
                                     const int* __restrict__ cu_tokens, const float* __restrict__ decay,
                                     float* __restrict__ sums, int heads, int dk, int dv, int state_rows) {
  pdl_trigger();
  pdl_wait();
  const int entry = blockIdx.x, head = blockIdx.y;
  const int i = blockIdx.z * blockDim.x + threadIdx.x;
  if (i >= dk * dv) return;
  const int slot = slots[entry];
  const int count = cu_tokens[entry + 1] - cu_tokens[entry];
  if (slot < 0 || slot >= state_rows || count <= 0) return;
  int first = 0;
  for (int e = 0; e < entry; ++e) first += (cu_tokens[e + 1] - cu_tokens[e] + LC - 1) / LC;
  const int chunks = (count + LC - 1) / LC;
  // decay^LC for whole chunks, decay^(tokens of the last chunk) for the last: two powers a thread
  const float whole = powf(decay[head], (float)LC);
  const float rest = powf(decay[head], (float)(count - (chunks - 1) * LC));
  float* cell = state + ((size_t)slot * heads + head) * dk * dv + i;
  float s = *cell;
  const size_t stride = (size_t)heads * dk * dv;
  float* sum = sums + ((size_t)first * heads + head) * dk * dv + i;
  for (int c0 = 0; c0 < chunks; c0 += 8) {               // eight chunks' sums are fetched before any is replaced
    float add[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) add[u] = c0 + u < chunks ? sum[(size_t)(c0 + u) * stride] : 0.f;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (c0 + u < chunks) {
        sum[(size_t)(c0 + u) * stride] = s;              // the state this chunk starts from
        s = fmaf(c0 + u + 1 < chunks ? whole : rest, s, add[u]);
      }
    }
  }
  *cell = s;
}

template <typename TI>
__global__ void __launch_bounds__(256)
lr_chunk_state_kernel(const TI* __restrict__ proj, int ld, int q_off, int act, const int* __restrict__ cu_tokens,
                      int entries, const float* __restrict__ decay, float* __restrict__ out,
                      const float* __restrict__ sums, int heads, int dk, int dv) {
  extern __shared__ __align__(16) float smem[];
  float* qs = smem;                       // [LC][dk]
  float* ss = qs + LC * dk;               // [dk][dv]
  float* pw = ss + dk * dv;               // [LC + 1]
  pdl_trigger();
  pdl_wait();
  int entry, local, first;
  if (!lr_locate(cu_tokens, entries, blockIdx.x, &entry, &local, &first)) return;
  const int head = blockIdx.y;
  const int t0 = cu_tokens[entry] + local * LC;
  const int len = min(LC, cu_tokens[entry + 1] - t0);
  const float lam = decay[head];
  for (int i = threadIdx.x; i <= LC; i += blockDim.x) pw[i] = powf(lam, (float)i);
#pragma unroll 8
  for (int i = threadIdx.x; i < LC * dk; i += blockDim.x) {
    const int t = i / dk, d = i - t * dk;
    qs[i] = t < len ? lr_act(to_float(proj[(size_t)(t0 + t) * ld + q_off + (size_t)head * dk + d]), act) : 0.f;
  }
  const float* src = sums + ((size_t)blockIdx.x * heads + head) * dk * dv;
#pragma unroll 8
  for (int i = threadIdx.x * 4; i < dk * dv; i += blockDim.x * 4)
    *reinterpret_cast<float4*>(ss + i) = *reinterpret_cast<const float4*>(src + i);
  __syncthreads();
  const int dv4 = dv >> 2;
  for (int item = threadIdx.x; item < 32 * dv4; item += blockDim.x) {
    const int tp = item / dv4, c = (item - tp * dv4) * 4;
    const int t1 = tp, t2 = tp + 32;
    if (t1 >= len) continue;
    float o1[4] = {0.f, 0.f, 0.f, 0.f}, o2[4] = {0.f, 0.f, 0.f, 0.f};
    const float* q1 = qs + t1 * dk;
    const float* q2 = qs + t2 * dk;
    for (int r = 0; r < dk; ++r) {
      const float4 s4 = *reinterpret_cast<const float4*>(ss + r * dv + c);
      fma4(o1, q1[r], s4);
      fma4(o2, q2[r], s4);
    }
    float had[4];
    float* dst = out + (size_t)(t0 + t1) * heads * dv + (size_t)head * dv + c;
    load4(dst, had);
#pragma unroll
    for (int e = 0; e < 4; ++e) had[e] = fmaf(pw[t1 + 1], o1[e], had[e]);
    store4(dst, had);
    if (t2 < len) {
      dst = out + (size_t)(t0 + t2) * heads * dv + (size_t)head * dv + c;
      load4(dst, had);
#pragma unroll
      for (int e = 0; e < 4; ++e) had[e] = fmaf(pw[t2 + 1], o2[e], had[e]);
      store4(dst, had);
    }
  }
}

// Chunks of LC tokens a step of these sizes has at most, and floats of workspace per chunk.
FE_EXPORT int fe_linear_recurrence_chunks(int n_tokens, int entries) { return (n_tokens + LC - 1) / LC + entries; }

FE_EXPORT int fe_linear_recurrence_chunked(const void* proj, int dtype, int ld, int q_off, int k_off, int v_off, int act,
                                           float* state, const int* slots, const int* cu_tokens, const float* decay,
                                           float* out, float* sums, int n_tokens, int entries, int heads, int dk, int dv,
                                           int state_rows, cudaStream_t stream) {
  if (entries <= 0 || n_tokens <= 0) return 0;
  if (dk < 1 || dv < 1 || heads > 65535 || entries > 65535) return FE_ERR_BAD_SHAPE;
  const int chunks = fe_linear_recurrence_chunks(n_tokens, entries);
  const size_t smem1 = sizeof(float) * ((size_t)LC * dk + (size_t)dk * LCP + (size_t)LC * dv + LC * LCP + LC + 4);
  const size_t smem3 = sizeof(float) * ((size_t)LC * dk + (size_t)dk * dv + LC + 4);
  if (smem1 > 200 * 1024 || smem3 > 200 * 1024) return FE_ERR_TOO_LARGE;
  if (dv % 4 || (uintptr_t)out % 16 || (uintptr_t)sums % 16) return FE_ERR_BAD_ALIGN;
  int rc = 0;
#define CHUNKED(TI)                                                                                                   \
  do {                                                                                                                \
    cudaFuncSetAttribute(lr_chunk_local_kernel<TI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);        \
    cudaFuncSetAttribute(lr_chunk_state_kernel<TI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem3);        \
    rc = fe_launch_dependent(lr_chunk_local_kernel<TI>, dim3(chunks, heads), dim3(256), smem1, stream,               \
                             (const TI*)proj, ld, q_off, k_off, v_off, act, cu_tokens, entries, decay, out, sums,     \
                             heads, dk, dv);                                                                          \
    if (rc == 0)                                                                                                      \
      rc = fe_launch_dependent(lr_chunk_scan_kernel, dim3(entries, heads, (dk * dv + 255) / 256), dim3(256), 0,      \
                               stream, state, slots, cu_tokens, decay, sums, heads, dk, dv, state_rows);             \
    if (rc == 0)                                                                                                      \
      rc = fe_launch_dependent(lr_chunk_state_kernel<TI>, dim3(chunks, heads), dim3(256), smem3, stream,             \
                               (const TI*)proj, ld, q_off, act, cu_tokens, entries, decay, out, sums, heads, dk, dv); \
  } while (0)
  if (dtype == FE_DTYPE_F32) CHUNKED(float);
  else if (dtype == FE_DTYPE_BF16) CHUNKED(bf16);
  else return FE_ERR_BAD_DTYPE;
#undef CHUNKED
  return rc ? rc : fe_last_error();
}
