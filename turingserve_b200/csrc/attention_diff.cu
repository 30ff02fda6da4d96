// Differential attention over the paged cache: every query head has TWO score maps over the same
// values.  A projection row holds, head by head, [q map 1 (D) | q map 2 (D)]; a cached key row holds
// [k map 1 (D) | k map 2 (D)] per kv head (2 D wide), a cached value row V values per kv head.  For a
// query at position p and keys j <= p:
//     a_m = softmax_j(q_m . k_m,j * scale) V      (m = 1, 2; 32-bit scores, weights and sums)
//     o   = a_1 - lambda * a_2;   out = o / sqrt(mean(o^2) + eps) * out_scale        (per head, over V)
// Query head h reads kv head h / (H / KVH).  No positions enter the scores.
//
// ts_kv_write_pair puts the step's new key and value rows (of different widths) into their pages.
// ts_attention_diff is the any-size kernel (32-bit arithmetic, float or bfloat16 storage): one block per
// (tile of ROWS query rows, kv head, request), a row being one (token, head-in-group) pair; keys come
// 32 at a time, lane j scores key j for both maps, the warp updates two online softmaxes, each lane
// accumulates its share of the V output columns for both maps.
#include "common.cuh"

namespace {

template <typename T>
__global__ void kv_write_pair_kernel(const T* __restrict__ proj, int proj_stride, int k_off, int v_off,
                                     T* __restrict__ k_cache, T* __restrict__ v_cache, const int* __restrict__ slots,
                                     int KVH, int DK, int DV, int page) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int slot = slots[t];
  if (slot < 0) return;
  const int pg = slot / page, in = slot % page;
  const T* row = proj + (size_t)t * proj_stride;
  for (int i = threadIdx.x; i < KVH * DK; i += blockDim.x) {
    const int g = i / DK, d = i % DK;
    k_cache[(((size_t)pg * KVH + g) * page + in) * DK + d] = row[k_off + i];
  }
  for (int i = threadIdx.x; i < KVH * DV; i += blockDim.x) {
    const int g = i / DV, d = i % DV;
    v_cache[(((size_t)pg * KVH + g) * page + in) * DV + d] = row[v_off + i];
  }
}

constexpr int ROWS = 16;
constexpr int KT = 32;
constexpr int NWARPS = 4;
constexpr int RPW = ROWS / NWARPS;
constexpr int MAX_VPL = 8;      // V <= 256

template <typename T>
__global__ void __launch_bounds__(NWARPS * 32)
attention_diff_kernel(T* __restrict__ out, const T* __restrict__ proj, int proj_stride,
                      const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                      const int* __restrict__ block_tables, const int* __restrict__ q_start,
                      const int* __restrict__ seq_lens, int table_width, int H, int KVH, int D, int V, int page,
                      float scale, float lambda, float eps, float out_scale) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float smem[];
  const int b = blockIdx.z, kvh = blockIdx.y;
  const int G = H / KVH;
  const int qs = q_start[b];
  const int q_len = q_start[b + 1] - qs;
  const int seq_len = seq_lens[b];
  const int row0 = blockIdx.x * ROWS;
  const int n_rows = q_len * G;
  if (row0 >= n_rows) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int vpl = (V + 31) / 32;
  const int prefix = seq_len - q_len;
  const int D2 = 2 * D;

  float* q_s = smem;                          // [ROWS][2D]
  float* k_s = q_s + ROWS * D2;               // [KT][2D+1]
  float* v_s = k_s + KT * (D2 + 1);           // [KT][V]
  __shared__ size_t key_page[KT];

  for (int idx = threadIdx.x; idx < ROWS * D2; idx += blockDim.x) {
    const int r = idx / D2, d = idx % D2;
    const int row = row0 + r;
    float v = 0.f;
    if (row < n_rows) {
      const int t = row / G, g = row % G;
      v = to_f(proj[(size_t)(qs + t) * proj_stride + (size_t)(kvh * G + g) * D2 + d]);
    }
    q_s[idx] = v;
  }

  const int last_row = min(row0 + ROWS, n_rows) - 1;
  const int j_hi = prefix + last_row / G;

  float m[RPW][2], l[RPW][2], acc[RPW][2][MAX_VPL];
  int p_row[RPW];
#pragma unroll
  for (int r = 0; r < RPW; ++r) {
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      m[r][c] = -INFINITY;
      l[r][c] = 0.f;
#pragma unroll
      for (int i = 0; i < MAX_VPL; ++i) acc[r][c][i] = 0.f;
    }
    const int row = row0 + warp * RPW + r;
    p_row[r] = (row < n_rows) ? prefix + row / G : -1;
  }

  if (seq_len > 0 && j_hi >= 0) {
    for (int j0 = 0; j0 <= j_hi; j0 += KT) {
      __syncthreads();
      if (threadIdx.x < KT) {
        const int j = j0 + threadIdx.x;
        size_t off = 0;
        if (j <= j_hi) {
          const int pg = block_tables[(size_t)b * table_width + j / page];
          off = ((size_t)pg * KVH + kvh) * page + (size_t)(j % page);
        }
        key_page[threadIdx.x] = off;
      }
      __syncthreads();
      for (int idx = threadIdx.x; idx < KT * D2; idx += blockDim.x) {
        const int kk = idx / D2, d = idx % D2;
        k_s[kk * (D2 + 1) + d] = (j0 + kk <= j_hi) ? to_f(k_cache[key_page[kk] * D2 + d]) : 0.f;
      }
      for (int idx = threadIdx.x; idx < KT * V; idx += blockDim.x) {
        const int kk = idx / V, d = idx % V;
        v_s[idx] = (j0 + kk <= j_hi) ? to_f(v_cache[key_page[kk] * V + d]) : 0.f;
      }
      __syncthreads();
      const int j = j0 + lane;
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        if (p_row[r] < j0) continue;                 // the whole tile lies in this row's future (warp-uniform)
        const bool ok = j <= p_row[r];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const float* qr = q_s + (warp * RPW + r) * D2 + c * D;
          const float* kr = k_s + lane * (D2 + 1) + c * D;
          float s = 0.f;
          for (int d = 0; d < D; ++d) s = fmaf(qr[d], kr[d], s);
          s = ok ? s * scale : -INFINITY;
          const float m_new = fmaxf(m[r][c], warp_max(s));   // j0 <= p_row: key j0 is visible, so m_new is finite
          const float p = ok ? expf(s - m_new) : 0.f;
          const float corr = (m[r][c] == -INFINITY) ? 0.f : expf(m[r][c] - m_new);
          l[r][c] = l[r][c] * corr + warp_sum(p);
          m[r][c] = m_new;
#pragma unroll
          for (int i = 0; i < MAX_VPL; ++i) acc[r][c][i] *= corr;
          for (int kk = 0; kk < KT; ++kk) {
            const float pk = __shfl_sync(0xffffffffu, p, kk);
            const float* vr = v_s + kk * V;
#pragma unroll
            for (int i = 0; i < MAX_VPL; ++i) {
              const int d = lane + 32 * i;
              if (i < vpl && d < V) acc[r][c][i] = fmaf(pk, vr[d], acc[r][c][i]);
            }
          }
        }
      }
    }
  }

#pragma unroll
  for (int r = 0; r < RPW; ++r) {
    const int row = row0 + warp * RPW + r;
    if (row >= n_rows) continue;                     // warp-uniform
    const int t = row / G, g = row % G;
    const float i1 = l[r][0] > 0.f ? 1.f / l[r][0] : 0.f;
    const float i2 = l[r][1] > 0.f ? 1.f / l[r][1] : 0.f;
    float o[MAX_VPL];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_VPL; ++i) {
      const int d = lane + 32 * i;
      o[i] = (i < vpl && d < V) ? acc[r][0][i] * i1 - lambda * (acc[r][1][i] * i2) : 0.f;
      ss += o[i] * o[i];
    }
    ss = warp_sum(ss);
    const float f = out_scale / sqrtf(ss / (float)V + eps);
    T* dst = out + (size_t)(qs + t) * H * V + (size_t)(kvh * G + g) * V;
#pragma unroll
    for (int i = 0; i < MAX_VPL; ++i) {
      const int d = lane + 32 * i;
      if (i < vpl && d < V) dst[d] = from_f<T>(o[i] * f);
    }
  }
}

template <typename T>
int launch_diff(void* out, const void* proj, int proj_stride, const void* k_cache, const void* v_cache,
                const int* block_tables, const int* q_start, const int* seq_lens, int B, int table_width,
                int max_q_len, int H, int KVH, int D, int V, int page, float scale, float lambda, float eps,
                float out_scale, cudaStream_t s) {
  const int G = H / KVH;
  const size_t smem = sizeof(float) * ((size_t)ROWS * 2 * D + (size_t)KT * (2 * D + 1) + (size_t)KT * V);
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_diff_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) TS_REFUSE((int)e, "ts_attention_diff: shared memory %zu: %s", smem, cudaGetErrorString(e));
    configured = smem;
  }
  dim3 grid(ceil_div(max_q_len * G, ROWS), KVH, B);
  ts_launch(attention_diff_kernel<T>, dim3(grid), dim3(NWARPS * 32), smem, s, (T*)out, (const T*)proj, proj_stride,
            (const T*)k_cache, (const T*)v_cache, block_tables, q_start, seq_lens, table_width, H, KVH, D, V, page,
            scale, lambda, eps, out_scale);
  TS_LAUNCH_CHECK();
}

}  // namespace

// proj rows: keys at column k_off (KVH x DK), values at v_off (KVH x DV).  Caches [pages, KVH, page, DK|DV].
TS_API int ts_kv_write_pair(const void* proj, int proj_stride, int k_off, int v_off, void* k_cache, void* v_cache,
                            const int* slots, int T, int KVH, int DK, int DV, int page, int dtype, void* stream) {
  if (T <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TS_F32)
    ts_launch(kv_write_pair_kernel<float>, dim3(T), dim3(128), 0, s, (const float*)proj, proj_stride, k_off, v_off,
              (float*)k_cache, (float*)v_cache, slots, KVH, DK, DV, page);
  else if (dtype == TS_BF16)
    ts_launch(kv_write_pair_kernel<bf16>, dim3(T), dim3(128), 0, s, (const bf16*)proj, proj_stride, k_off, v_off,
              (bf16*)k_cache, (bf16*)v_cache, slots, KVH, DK, DV, page);
  else
    TS_REFUSE(TS_ERR_DTYPE, "ts_kv_write_pair: dtype %d", dtype);
  TS_LAUNCH_CHECK();
}

// proj rows: the queries at column 0, H x [map 1 (D) | map 2 (D)].  k_cache rows are 2 D wide, v_cache rows V.
TS_API int ts_attention_diff(void* out, const void* proj, int proj_stride, const void* k_cache, const void* v_cache,
                             const int* block_tables, const int* q_start, const int* seq_lens, int B,
                             int table_width, int max_q_len, int H, int KVH, int D, int V, int page, float scale,
                             float lambda, float eps, float out_scale, int dtype, void* stream) {
  if (B <= 0 || max_q_len <= 0) return 0;
  if (KVH <= 0 || H % KVH) TS_REFUSE(TS_ERR_SHAPE, "ts_attention_diff: %d heads over %d kv heads", H, KVH);
  if (D <= 0 || D > 256 || V <= 0 || V > 32 * MAX_VPL)
    TS_REFUSE(TS_ERR_LIMIT, "ts_attention_diff: maps of %d, values of %d (limits 256, %d)", D, V, 32 * MAX_VPL);
  if (B > 65535 || KVH > 65535) TS_REFUSE(TS_ERR_LIMIT, "ts_attention_diff: %d requests / %d kv heads per launch", B, KVH);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TS_F32)
    return launch_diff<float>(out, proj, proj_stride, k_cache, v_cache, block_tables, q_start, seq_lens, B, table_width,
                              max_q_len, H, KVH, D, V, page, scale, lambda, eps, out_scale, s);
  if (dtype == TS_BF16)
    return launch_diff<bf16>(out, proj, proj_stride, k_cache, v_cache, block_tables, q_start, seq_lens, B, table_width,
                             max_q_len, H, KVH, D, V, page, scale, lambda, eps, out_scale, s);
  TS_REFUSE(TS_ERR_DTYPE, "ts_attention_diff: dtype %d", dtype);
}
