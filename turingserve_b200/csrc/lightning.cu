// Linear attention with a per-head decay ("lightning attention"): for every request and head a matrix
// state S [D, V] in 32-bit that lives in a state slot between steps,
//     S_t = lam_h S_{t-1} + k_t v_t^T,     o_t = S_t^T q_t,
// with q, k, v = act(projection) taken from one fused projection row [q (H D) | k (H D) | v (H V) | ...].
// The activation (SiLU) is applied here, rounded to the storage type as the projection's own epilogue
// would round it; everything from there on (products with the state, decay, the state itself, the
// output) is 32-bit.  Output: 32-bit rows [T, H V] (a norm over all heads follows in another kernel).
//
// ts_lightning runs the tokens of a step in order: one block per (head, request); thread j owns column
// j of the state.  A request's only token (decoding) updates the state in place in global memory; a
// portion keeps the state in shared memory over its tokens, which arrive in groups of LT_GROUP rows
// staged in shared memory.
#include "common.cuh"

namespace {

constexpr int LT_GROUP = 16;

template <typename T> __device__ __forceinline__ float act_silu(float z) { return round_to<T>(z / (1.f + expf(-z))); }

template <typename T>
__global__ void __launch_bounds__(256)
lightning_kernel(float* __restrict__ out, const T* __restrict__ proj, int proj_stride, float* __restrict__ state,
                 const float* __restrict__ decay, const int* __restrict__ q_start, const int* __restrict__ slots,
                 int H, int D, int V, int state_in_smem) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float smem[];
  const int h = blockIdx.x, b = blockIdx.y;
  const int t0 = q_start[b], n = q_start[b + 1] - t0;
  if (n <= 0) return;
  const float lam = decay[h];
  float* S = state + ((size_t)slots[b] * H + h) * D * V;
  float* q_s = smem;                       // [LT_GROUP][D]
  float* k_s = q_s + LT_GROUP * D;         // [LT_GROUP][D]
  float* v_s = k_s + LT_GROUP * D;         // [LT_GROUP][V]
  float* S_s = v_s + LT_GROUP * V;         // [D][V] when state_in_smem
  const bool staged = state_in_smem && n > 1;
  if (staged) {
    for (int i = threadIdx.x; i < D * V; i += blockDim.x) S_s[i] = S[i];
  }
  float* St = staged ? S_s : S;
  const int q_off = h * D, k_off = H * D + h * D, v_off = 2 * H * D + h * V;
  for (int g0 = 0; g0 < n; g0 += LT_GROUP) {
    const int gn = min(LT_GROUP, n - g0);
    __syncthreads();
    for (int i = threadIdx.x; i < gn * D; i += blockDim.x) {
      const int r = i / D, d = i % D;
      const T* row = proj + (size_t)(t0 + g0 + r) * proj_stride;
      q_s[i] = act_silu<T>(to_f(row[q_off + d]));
      k_s[i] = act_silu<T>(to_f(row[k_off + d]));
    }
    for (int i = threadIdx.x; i < gn * V; i += blockDim.x) {
      const int r = i / V, d = i % V;
      v_s[i] = act_silu<T>(to_f(proj[(size_t)(t0 + g0 + r) * proj_stride + v_off + d]));
    }
    __syncthreads();
    for (int j = threadIdx.x; j < V; j += blockDim.x) {
      for (int r = 0; r < gn; ++r) {
        const float vj = v_s[r * V + j];
        const float* qr = q_s + r * D;
        const float* kr = k_s + r * D;
        float o = 0.f;
#pragma unroll 4
        for (int i = 0; i < D; ++i) {
          const float s = fmaf(lam, St[i * V + j], kr[i] * vj);
          St[i * V + j] = s;
          o = fmaf(s, qr[i], o);
        }
        out[(size_t)(t0 + g0 + r) * H * V + h * V + j] = o;
      }
    }
  }
  if (staged) {
    __syncthreads();
    for (int i = threadIdx.x; i < D * V; i += blockDim.x) S[i] = S_s[i];
  }
}

}  // namespace

// proj: [T, proj_stride] rows holding q at column 0, k at H D, v at 2 H D.  state: [slots, H, D, V] 32-bit.
// decay: [H] 32-bit on the device.  out: [T, H V] 32-bit.
TS_API int ts_lightning(float* out, const void* proj, int proj_stride, float* state, const float* decay,
                        const int* q_start, const int* slots, int B, int H, int D, int V, int dtype, void* stream) {
  if (B <= 0) return 0;
  if (H <= 0 || D <= 0 || V <= 0) TS_REFUSE(TS_ERR_SHAPE, "ts_lightning: %d heads of %d x %d", H, D, V);
  if (B > 65535) TS_REFUSE(TS_ERR_LIMIT, "ts_lightning: %d requests per launch", B);
  cudaStream_t s = (cudaStream_t)stream;
  const size_t group = sizeof(float) * LT_GROUP * (2 * (size_t)D + V);
  size_t smem = group + sizeof(float) * (size_t)D * V;
  int in_smem = 1;
  if (smem > 200 * 1024) {          // a state too large for shared memory stays in global memory (and in L2)
    smem = group;
    in_smem = 0;
  }
  if (group > 200 * 1024) TS_REFUSE(TS_ERR_LIMIT, "ts_lightning: heads of %d x %d are too wide", D, V);
  const int threads = V >= 256 ? 256 : (V + 31) / 32 * 32;
#define TS_LT(TT)                                                                                                   \
  do {                                                                                                              \
    static size_t configured = 0;                                                                                   \
    if (smem > 48 * 1024 && smem > configured) {                                                                    \
      cudaError_t e = cudaFuncSetAttribute(lightning_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) TS_REFUSE((int)e, "ts_lightning: shared memory %zu: %s", smem, cudaGetErrorString(e)); \
      configured = smem;                                                                                            \
    }                                                                                                               \
    ts_launch(lightning_kernel<TT>, dim3(H, B), dim3(threads), smem, s, out, (const TT*)proj, proj_stride, state, \
              decay, q_start, slots, H, D, V, in_smem);                                                             \
  } while (0)
  if (dtype == TS_F32) TS_LT(float);
  else if (dtype == TS_BF16) TS_LT(bf16);
  else TS_REFUSE(TS_ERR_DTYPE, "ts_lightning: dtype %d", dtype);
#undef TS_LT
  TS_LAUNCH_CHECK();
}
