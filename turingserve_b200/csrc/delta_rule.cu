// The gated delta rule: for every request and head a matrix memory M [D, V] in 32-bit that lives in a state slot
// between steps (S in the code).  Per token, with q and k of unit length (q also over sqrt(D)), a fade d in (0, 1)
// (g in the code) and a write strength w in (0, 1) (beta):
//     M <- d M;   e = w (v - M^T k);   M <- M + k e^T;   y = M^T q          (y comes after the token's own write).
// q, k and v are a fused projection's columns after a causal filter of a few taps per channel and SiLU; the
// filter's last taps - 1 inputs are kept behind S in the same slot: [H D V | (taps - 1) x C], C = 2 G D + H V.
//
// Three kernels:
//   ts_delta_prepare      one block per (token, head): filter + SiLU, unit length per head, g, beta and k.q, as 32-bit
//                         rows [q (G D) | k (G D) | v (H V) | g (H) | beta (H) | k.q (G)]; reads the slot's filter
//                         inputs for the tokens before the step's first, writes nothing to the slot
//   ts_delta_scan         the recurrence, token by token for portions and single tokens alike (cutting a prompt
//                         changes no bit); afterwards the request's blocks store the filter's new last inputs
//   ts_head_gated_rmsnorm o / rms(o) per head, times a weight shared by the heads, times silu(gate)
//
// The scan: one pass over the state per token.  With a = (g S)^T k and c = (g S)^T q, both sums over the old
// state, u = beta (v - a) and o = c + (k.q) u, so the read-out needs no second pass after the write.  A column
// of S is independent of the others: P lanes of one warp hold it (R rows each, in registers over all tokens of
// the step), the two sums cross the P lanes by shuffles, and no block-wide barrier sits inside a token.  Tokens
// arrive in groups of DR_GROUP rows by cp.async, three groups ahead of the one that is computed.
#include "common.cuh"
#include "mma_utils.cuh"

namespace {

constexpr int DR_GROUP = 16;     // tokens staged at a time
constexpr int DR_STAGES = 4;     // groups in flight or in use: the rows of three groups are on their way while one is computed
constexpr int DR_PAD = 4;        // floats between two lanes' row pieces in shared memory (bank spread)

__device__ __forceinline__ void cp_async_4(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

template <typename T>
__global__ void __launch_bounds__(128)
delta_prepare_kernel(float* __restrict__ ready, const T* __restrict__ proj, int proj_stride,
                     const float* __restrict__ conv_w, const float* __restrict__ a_log,
                     const float* __restrict__ dt_bias, const float* __restrict__ state, size_t state_stride,
                     const int* __restrict__ token_request, const int* __restrict__ q_start,
                     const int* __restrict__ slots, int H, int G, int D, int V, int taps, float unit_eps) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float f_s[];                       // [2 D] filtered and activated q and k of one head
  __shared__ float scratch[32];
  const int t = blockIdx.x, unit = blockIdx.y;         // units: the G query/key heads, then the H value heads
  const int b = token_request[t];
  const int t0 = q_start[b], i = t - t0;
  const int qk = G * D, hv = H * V, C = 2 * qk + hv, W = C + 2 * H + G;
  const float* tail = state + (size_t)slots[b] * state_stride + (size_t)H * D * V;     // [taps - 1][C]
  float* out = ready + (size_t)t * W;
  auto filtered = [&](int c) {
    float acc = 0.f;
    for (int u = 0; u < taps; ++u) {
      const int rel = i - (taps - 1) + u;              // the input's place, counted from the step's first token
      const float x = rel >= 0 ? to_f(proj[(size_t)(t0 + rel) * proj_stride + c]) : tail[(size_t)(rel + taps - 1) * C + c];
      acc = fmaf(conv_w[c * taps + u], x, acc);
    }
    return acc / (1.f + expf(-acc));
  };
  if (unit >= G) {
    const int h = unit - G;
    for (int d = threadIdx.x; d < V; d += blockDim.x) out[2 * qk + h * V + d] = filtered(2 * qk + h * V + d);
    if (h == 0) {
      for (int hh = threadIdx.x; hh < H; hh += blockDim.x) {
        const T* row = proj + (size_t)t * proj_stride + C + hv;
        const float bb = to_f(row[hh]), aa = to_f(row[H + hh]);
        out[C + hh] = expf(-expf(a_log[hh]) * softplus_f(aa + dt_bias[hh]));
        out[C + H + hh] = 1.f / (1.f + expf(-bb));
      }
    }
    return;
  }
  const int g = unit;
  float sq = 0.f, sk = 0.f, dot = 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const float fq = filtered(g * D + d), fk = filtered(qk + g * D + d);
    f_s[d] = fq;
    f_s[D + d] = fk;
    sq = fmaf(fq, fq, sq);
    sk = fmaf(fk, fk, sk);
    dot = fmaf(fq, fk, dot);
  }
  sq = block_sum(sq, scratch);
  sk = block_sum(sk, scratch);
  dot = block_sum(dot, scratch);
  const float rq = 1.f / (sqrtf((float)D) * sqrtf(sq + unit_eps)), rk = 1.f / sqrtf(sk + unit_eps);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {  // (a thread reads back what it wrote itself)
    out[g * D + d] = f_s[d] * rq;
    out[qk + g * D + d] = f_s[D + d] * rk;
  }
  if (threadIdx.x == 0) out[C + 2 * H + g] = dot * rq * rk;
}

// R rows of a column a lane; P lanes a column; CW = 32 / P columns a warp.
template <int R>
__global__ void __launch_bounds__(256, 1)
delta_scan_kernel(float* __restrict__ out, const float* __restrict__ ready, const void* __restrict__ proj,
                  int proj_stride, int proj_is_bf16, float* __restrict__ state, size_t state_stride,
                  const int* __restrict__ q_start, const int* __restrict__ slots, int H, int G, int D, int V,
                  int taps, int P, int vec4, int group) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float smem[];
  const int h = blockIdx.y, b = blockIdx.z;
  const int t0 = q_start[b], n = q_start[b + 1] - t0;
  if (n <= 0) return;
  const int kvh = h / (H / G);
  const int qk = G * D, hv = H * V, C = 2 * qk + hv, W = C + 2 * H + G;
  const int CW = 32 / P;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int p = lane / CW, cw = lane % CW;
  const int cols_block = nwarps * CW;
  const int col = warp * CW + cw;                              // within the block
  const int j = blockIdx.x * cols_block + col;
  const bool live = j < V;
  const int row_w = P * (R + DR_PAD);                          // floats of one token's q (or k) in shared memory
  const int tok_w = 2 * row_w + ((cols_block + 3 + 3) & ~3);   // q | k | v of the block's columns | g, beta, k.q (16-byte rows)
  float* base = state + (size_t)slots[b] * state_stride;
  float* S = base + (size_t)h * D * V;

  float s[R];
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int d = p * R + i;
    s[i] = (live && d < D) ? S[(size_t)d * V + j] : 0.f;
  }
  for (int i = threadIdx.x; i < DR_STAGES * group * tok_w; i += blockDim.x) smem[i] = 0.f;   // (rows beyond D stay zero)
  __syncthreads();

  // a warp brings whole tokens, its lanes the pieces of a row: additions and shifts only (a lane's copies follow one
  // another in a chain of dependent index arithmetic, so a division per copy would cost more than the scan itself)
  auto fetch = [&](int g0, int buf) {
    const int gn = min(group, n - g0);
    float* dst0 = smem + (size_t)buf * group * tok_w;
    for (int r = warp; r < gn; r += nwarps) {
      const float* row = ready + (size_t)(t0 + g0 + r) * W;
      const float* qrow = row + kvh * D;
      const float* krow = row + qk + kvh * D;
      float* dst = dst0 + r * tok_w;
      if (vec4) {
        for (int d = lane * 4; d < D; d += 128) {
          const int off = (d / R) * (R + DR_PAD) + d % R;          // (R is a power of two)
          cp_async_16(dst + off, qrow + d, true);
          cp_async_16(dst + row_w + off, krow + d, true);
        }
      } else {
        for (int d = lane; d < D; d += 32) {
          const int off = (d / R) * (R + DR_PAD) + d % R;
          cp_async_4(dst + off, qrow + d);
          cp_async_4(dst + row_w + off, krow + d);
        }
      }
      float* tail_dst = dst + 2 * row_w;
      for (int c = lane; c < cols_block + 3; c += 32) {
        if (c < cols_block) {
          const int jj = blockIdx.x * cols_block + c;
          if (jj < V) cp_async_4(tail_dst + c, row + 2 * qk + h * V + jj);
        } else if (c == cols_block) cp_async_4(tail_dst + c, row + C + h);
        else if (c == cols_block + 1) cp_async_4(tail_dst + c, row + C + H + h);
        else cp_async_4(tail_dst + c, row + C + 2 * H + kvh);
      }
    }
  };

#pragma unroll
  for (int st = 0; st < DR_STAGES - 1; ++st) {
    if (st * group < n) fetch(st * group, st);
    cp_async_commit();
  }
  int buf = 0;
  for (int g0 = 0; g0 < n; g0 += group, buf = (buf + 1) % DR_STAGES) {
    const int gn = min(group, n - g0);
    // (the buffer filled now is the one the group before this one was computed from: the barrier at its end freed it)
    if (g0 + (DR_STAGES - 1) * group < n) fetch(g0 + (DR_STAGES - 1) * group, (buf + DR_STAGES - 1) % DR_STAGES);
    cp_async_commit();
    cp_async_wait<DR_STAGES - 1>();
    __syncthreads();                                           // this group's rows are here
    const float* grp = smem + (size_t)buf * group * tok_w;
    for (int r = 0; r < gn; ++r) {
      const float* tok = grp + r * tok_w;
      const float4* qr = reinterpret_cast<const float4*>(tok + p * (R + DR_PAD));
      const float4* kr = reinterpret_cast<const float4*>(tok + row_w + p * (R + DR_PAD));
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, c0 = 0.f, c1 = 0.f, c2 = 0.f, c3 = 0.f;   // eight chains of R / 4
#pragma unroll
      for (int i = 0; i < R / 4; ++i) {
        const float4 k4 = kr[i], q4 = qr[i];
        a0 = fmaf(s[4 * i + 0], k4.x, a0);
        c0 = fmaf(s[4 * i + 0], q4.x, c0);
        a1 = fmaf(s[4 * i + 1], k4.y, a1);
        c1 = fmaf(s[4 * i + 1], q4.y, c1);
        a2 = fmaf(s[4 * i + 2], k4.z, a2);
        c2 = fmaf(s[4 * i + 2], q4.z, c2);
        a3 = fmaf(s[4 * i + 3], k4.w, a3);
        c3 = fmaf(s[4 * i + 3], q4.w, c3);
      }
      float a = (a0 + a1) + (a2 + a3), c = (c0 + c1) + (c2 + c3);
      for (int off = CW; off < 32; off <<= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, off);
        c += __shfl_xor_sync(0xffffffffu, c, off);
      }
      const float* sc = tok + 2 * row_w + cols_block;
      const float g = sc[0], beta = sc[1], kq = sc[2];
      const float u = beta * (tok[2 * row_w + col] - g * a);
      const float o = fmaf(kq, u, g * c);
#pragma unroll
      for (int i = 0; i < R / 4; ++i) {
        const float4 k4 = kr[i];
        s[4 * i + 0] = fmaf(k4.x, u, g * s[4 * i + 0]);
        s[4 * i + 1] = fmaf(k4.y, u, g * s[4 * i + 1]);
        s[4 * i + 2] = fmaf(k4.z, u, g * s[4 * i + 2]);
        s[4 * i + 3] = fmaf(k4.w, u, g * s[4 * i + 3]);
      }
      if (p == 0 && live) out[(size_t)(t0 + g0 + r) * hv + h * V + j] = o;
    }
    __syncthreads();                                           // the buffer may be filled again
  }
  cp_async_wait<0>();
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int d = p * R + i;
    if (live && d < D) S[(size_t)d * V + j] = s[i];
  }
  // the filter's new last inputs: what the slot held, moved up by n, then this step's raw rows
  if (taps > 1) {
    float* tail = base + (size_t)H * D * V;
    const int first = (h * gridDim.x + blockIdx.x) * blockDim.x + threadIdx.x, stride = H * gridDim.x * blockDim.x;
    for (int c = first; c < C; c += stride) {                  // every block of the request takes a share of the channels
      float nv[7];
#pragma unroll
      for (int jt = 0; jt < 7; ++jt) {
        const int rel = n - (taps - 1) + jt;
        nv[jt] = 0.f;
        if (jt < taps - 1) {
          if (rel >= 0) {
            const size_t at = (size_t)(t0 + rel) * proj_stride + c;
            nv[jt] = proj_is_bf16 ? to_f(reinterpret_cast<const bf16*>(proj)[at]) : reinterpret_cast<const float*>(proj)[at];
          } else {
            nv[jt] = tail[(size_t)(rel + taps - 1) * C + c];
          }
        }
      }
#pragma unroll
      for (int jt = 0; jt < 7; ++jt)
        if (jt < taps - 1) tail[(size_t)jt * C + c] = nv[jt];
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
head_gated_rmsnorm_kernel(T* __restrict__ out, const float* __restrict__ x, const T* __restrict__ gate, int gate_stride,
                          const float* __restrict__ w, float eps, int H, int V) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int h = blockIdx.y * nwarps + warp; h < H; h += gridDim.y * nwarps) {      // a warp a head
    const float* xr = x + ((size_t)t * H + h) * V;
    const T* gr = gate + (size_t)t * gate_stride + (size_t)h * V;
    float ss = 0.f;
    for (int i = lane; i < V; i += 32) ss = fmaf(xr[i], xr[i], ss);
    ss = warp_sum(ss);
    const float rstd = 1.f / sqrtf(ss / (float)V + eps);
    for (int i = lane; i < V; i += 32) {
      const float z = to_f(gr[i]);
      out[((size_t)t * H + h) * V + i] = from_f<T>(xr[i] * rstd * w[i] * (z / (1.f + expf(-z))));
    }
  }
}

int g_delta_rows = 0;

}  // namespace

// Rows of a state column a lane of the scan holds (8, 16 or 32; 0: by the key width).  For measurements.
TS_API void ts_set_delta_rows(int rows) { g_delta_rows = rows; }

// ready: [T, 2 G D + H V + 2 H + G] 32-bit.  proj: [T, proj_stride] rows holding q at column 0, k at G D, v at
// 2 G D, then the gate (H V), b (H) and a (H).  conv_w: [2 G D + H V, taps] 32-bit.  state: [slots, state_stride].
TS_API int ts_delta_prepare(float* ready, const void* proj, int proj_stride, const float* conv_w, const float* a_log,
                            const float* dt_bias, const float* state, long long state_stride, const int* token_request,
                            const int* q_start, const int* slots, int T, int H, int G, int D, int V, int taps,
                            float unit_eps, int dtype, void* stream) {
  if (T <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || D <= 0 || V <= 0) TS_REFUSE(TS_ERR_SHAPE, "ts_delta_prepare: %d heads over %d of %d x %d", H, G, D, V);
  if (taps < 1 || taps > 8) TS_REFUSE(TS_ERR_LIMIT, "ts_delta_prepare: %d taps (1 to 8)", taps);
  const size_t smem = sizeof(float) * (size_t)2 * D;
  if (smem > 200 * 1024) TS_REFUSE(TS_ERR_LIMIT, "ts_delta_prepare: keys of %d", D);
  if (G + H > 65535) TS_REFUSE(TS_ERR_LIMIT, "ts_delta_prepare: %d heads", G + H);
  cudaStream_t s = (cudaStream_t)stream;
#define TS_DP(TT)                                                                                                        \
  do {                                                                                                                   \
    static size_t configured = 0;                                                                                        \
    if (smem > 48 * 1024 && smem > configured) {                                                                         \
      cudaError_t e = cudaFuncSetAttribute(delta_prepare_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) TS_REFUSE((int)e, "ts_delta_prepare: shared memory %zu: %s", smem, cudaGetErrorString(e));   \
      configured = smem;                                                                                                 \
    }                                                                                                                    \
    ts_launch(delta_prepare_kernel<TT>, dim3(T, G + H), dim3(128), smem, s, ready, (const TT*)proj, proj_stride, conv_w, a_log, \
              dt_bias, state, (size_t)state_stride, token_request, q_start, slots, H, G, D, V, taps, unit_eps);          \
  } while (0)
  if (dtype == TS_F32) TS_DP(float);
  else if (dtype == TS_BF16) TS_DP(bf16);
  else TS_REFUSE(TS_ERR_DTYPE, "ts_delta_prepare: dtype %d", dtype);
#undef TS_DP
  TS_LAUNCH_CHECK();
}

// out: [T, H V] 32-bit.  proj: the raw projection rows (for the filter's new last inputs).  max_q_len: the most tokens a
// request of the launch brings (0: unknown); it sizes the staging buffers.
TS_API int ts_delta_scan(float* out, const float* ready, const void* proj, int proj_stride, float* state,
                         long long state_stride, const int* q_start, const int* slots, int B, int H, int G, int D, int V,
                         int taps, int max_q_len, int dtype, void* stream) {
  if (B <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || D <= 0 || V <= 0) TS_REFUSE(TS_ERR_SHAPE, "ts_delta_scan: %d heads over %d of %d x %d", H, G, D, V);
  if (taps < 1 || taps > 8) TS_REFUSE(TS_ERR_LIMIT, "ts_delta_scan: %d taps (1 to 8)", taps);
  if (dtype != TS_F32 && dtype != TS_BF16) TS_REFUSE(TS_ERR_DTYPE, "ts_delta_scan: dtype %d", dtype);
  if (B > 65535 || H > 65535) TS_REFUSE(TS_ERR_LIMIT, "ts_delta_scan: %d requests / %d heads per launch", B, H);
  // rows of a column a lane holds: few rows mean more lanes a column, so more warps to hide one another's latencies
  // (one warp a scheduler waits out every dependent instruction), but a longer shuffle tree
  // tokens staged at a time: no request of the launch brings more than max_q_len (0: unknown)
  const int group = max_q_len > 0 ? min(DR_GROUP, max_q_len) : DR_GROUP;
  int R = g_delta_rows;
  // (single tokens: one trip through the chain, so the fewest threads a column, which fit the chip in one wave)
  if (R != 8 && R != 16 && R != 32) R = max_q_len == 1 ? 32 : (D <= 256 ? 8 : (D <= 512 ? 16 : 32));
  while (R < 32 && R * 32 < D) R *= 2;
  int P = 1;
  while (P * R < D) P <<= 1;
  if (P > 32) TS_REFUSE(TS_ERR_LIMIT, "ts_delta_scan: keys of %d (limit 1024)", D);
  const int CW = 32 / P;
  // 16 columns a block (or what a warp holds, if that is more): a portion of one request has H x V / 16 blocks to
  // spread over the chip, and every block stages the same q and k rows out of L2
  const int nwarps = max(1, min(8, min(ceil_div(16, CW), ceil_div(V, CW))));
  const int cols_block = nwarps * CW;
  const int W = 2 * G * D + H * V + 2 * H + G;
  const int vec4 = D % 4 == 0 && W % 4 == 0 && (G * D) % 4 == 0 && !((uintptr_t)ready & 15);
  const size_t smem = sizeof(float) * DR_STAGES * group * ((size_t)2 * P * (R + DR_PAD) + ((cols_block + 3 + 3) & ~3));
  if (smem > 200 * 1024) TS_REFUSE(TS_ERR_LIMIT, "ts_delta_scan: shared memory %zu", smem);
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(ceil_div(V, cols_block), H, B);
#define TS_DS(RR)                                                                                                        \
  do {                                                                                                                   \
    static size_t configured = 0;                                                                                        \
    if (smem > 48 * 1024 && smem > configured) {                                                                         \
      cudaError_t e = cudaFuncSetAttribute(delta_scan_kernel<RR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) TS_REFUSE((int)e, "ts_delta_scan: shared memory %zu: %s", smem, cudaGetErrorString(e));      \
      configured = smem;                                                                                                 \
    }                                                                                                                    \
    ts_launch(delta_scan_kernel<RR>, dim3(grid), dim3(nwarps * 32), smem, s, out, ready, proj, proj_stride,              \
              dtype == TS_BF16 ? 1 : 0, state, (size_t)state_stride, q_start, slots, H, G, D, V, taps, P, vec4, group);  \
  } while (0)
  if (R == 32) TS_DS(32);
  else if (R == 16) TS_DS(16);
  else TS_DS(8);
#undef TS_DS
  TS_LAUNCH_CHECK();
}

// out [T, H V] = x / sqrt(mean over a head's V of x^2 + eps) * w[V] * silu(gate); x 32-bit [T, H V]; gate rows
// gate_stride apart.
TS_API int ts_head_gated_rmsnorm(void* out, const float* x, const void* gate, int gate_stride, const float* w, float eps,
                                 int T, int H, int V, int dtype, void* stream) {
  if (T <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  // few tokens: the heads of a token spread over blocks of four warps; many: one block a token
  const int heads_y = T >= 512 ? 1 : min(ceil_div(H, 4), 65535);
  if (dtype == TS_F32)
    ts_launch(head_gated_rmsnorm_kernel<float>, dim3(T, heads_y), dim3(128), 0, s, (float*)out, x, (const float*)gate, gate_stride, w, eps, H, V);
  else if (dtype == TS_BF16)
    ts_launch(head_gated_rmsnorm_kernel<bf16>, dim3(T, heads_y), dim3(128), 0, s, (bf16*)out, x, (const bf16*)gate, gate_stride, w, eps, H, V);
  else
    TS_REFUSE(TS_ERR_DTYPE, "ts_head_gated_rmsnorm: dtype %d", dtype);
  TS_LAUNCH_CHECK();
}
