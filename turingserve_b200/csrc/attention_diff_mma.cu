// Differential attention (two score maps a head over the same values, see attention_diff.cu) on the
// tensor cores, bfloat16, for maps of D in {32, 64} and values of V in {64, 128}: prompt portions and
// single tokens alike, from the paged cache.
//
// Work split as the framework's softmax attention for prompt portions: one block per (tile of 64 query rows,
// kv head, request), a row being one (token, head-in-group) pair, so the G query heads of a kv head share
// every key/value tile; each of the 4 warps owns 16 rows (one m16n8k16 row block).  Keys come 64 at a
// time through a 3-stage cp.async pipeline into XOR-swizzled shared memory: a key row is 2 D wide
// ([map 1 | map 2]), a value row V.  For every tile a warp runs map 1 and then map 2: S = Q_m K_m^T, mask,
// online softmax (32-bit, exponentials in base 2), O_m += P V with P rounded to bfloat16 as an operand.
// At the end o = O_1 / l_1 - lambda O_2 / l_2, divided by its root mean square over V, times out_scale.
//
// A block whose rows all fit one warp (a request's single token, G <= 16) lets its four warps work for the
// SAME rows: warp w takes keys 16 w .. 16 w + 15 of every tile, and the four partial results (each with its own
// running maximum and sum) are merged through shared memory at the end, so a decoding request's keys are
// shared by four warps instead of waiting for one.  Such a request's keys are also cut over up to `max_splits`
// blocks (the grid's x index, which for a portion counts its row tiles): every block leaves its partial result
// in scratch, and the block that comes last for a (request, kv head) (a ticket counter; nobody waits) folds the
// partial results in split order and writes the output.
#include "common.cuh"
#include "mma_utils.cuh"

namespace {

constexpr int DM_WARPS = 4;
constexpr int DM_ROWS = DM_WARPS * 16;
constexpr int DM_TILE = 64;
constexpr int DM_STAGES = 3;
constexpr int DM_SPLIT_TILES = 4;         // fewest 64-key tiles a piece of a decoding request's keys holds
constexpr int DM_PAGES_S = 2048;          // block-table entries a block keeps in shared memory
constexpr float DM_LOG2E = 1.4426950408889634f;

template <int D, int V, bool SPLIT>
__global__ void __launch_bounds__(DM_WARPS * 32)
attention_diff_mma_kernel(bf16* __restrict__ out, const bf16* __restrict__ proj, int proj_stride,
                          const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                          const int* __restrict__ block_tables, const int* __restrict__ q_start,
                          const int* __restrict__ seq_lens, int table_width, int H, int KVH, int page, float scale,
                          float lambda, float eps, float out_scale, float* __restrict__ scratch,
                          int* __restrict__ counters, int max_splits) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int DK = 2 * D;                 // a cached key row
  constexpr int CHK = DK / 8, CHV = V / 8, KS = D / 16, NT = V / 8;
  constexpr int K_STAGE = DM_TILE * DK * 2, V_STAGE = DM_TILE * V * 2;
  extern __shared__ __align__(128) unsigned char smem[];
  const int b = blockIdx.z, kvh = blockIdx.y;
  const int G = H / KVH;
  const int qs = q_start[b];
  const int q_len = q_start[b + 1] - qs;
  const int seq_len = seq_lens[b];
  const int n_rows = q_len * G;
  const int n_row_tiles = (n_rows + DM_ROWS - 1) / DM_ROWS;
  // Two instances share a launch's requests: SPLIT takes those whose rows fit one warp (every warp then works for
  // rows 0..15 on its own 16 keys of every tile, with loops a quarter as long at compile time), the other the rest.
  constexpr bool split = SPLIT;
  if ((n_rows <= 16) != SPLIT) return;
  constexpr int NP = SPLIT ? 1 : DM_TILE / 16;                        // 16-key blocks of a tile a warp computes
  const int key0 = SPLIT ? (int)(threadIdx.x >> 5) * 16 : 0;          // where they start
  const int prefix = seq_len - q_len;
  // a split request: the grid's x index is the piece of its keys; a portion: its row tile
  int nsplit = 1;
  if (split && n_rows > 0 && scratch != nullptr) {
    const int all_tiles = seq_len > 0 ? (prefix + (n_rows - 1) / G) / DM_TILE + 1 : 0;
    // at least DM_SPLIT_TILES tiles a piece: every piece is one more partial result for the last block to fold
    nsplit = max(1, min(min((int)gridDim.x, max_splits), (all_tiles + DM_SPLIT_TILES - 1) / DM_SPLIT_TILES));
  }
  if ((int)blockIdx.x >= (split ? nsplit : n_row_tiles)) return;
  const int row0 = split ? 0 : (n_row_tiles - 1 - blockIdx.x) * DM_ROWS;      // longest tiles first
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int rw = split ? 0 : warp;

  unsigned char* k_s = smem;
  unsigned char* v_s = smem + DM_STAGES * K_STAGE;

  int pos[2];
  const bf16* qptr[2];
  bf16* optr[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = row0 + rw * 16 + (lane >> 2) + 8 * r;
    if (row < n_rows) {
      const int t = row / G, g = row % G;
      pos[r] = prefix + t;
      qptr[r] = proj + (size_t)(qs + t) * proj_stride + (size_t)(kvh * G + g) * DK;
      optr[r] = out + (size_t)(qs + t) * H * V + (size_t)(kvh * G + g) * V;
    } else {
      pos[r] = -1;
      qptr[r] = nullptr;
      optr[r] = nullptr;
    }
  }
  unsigned qf[2][KS][4];
  {
    const int kc = (lane & 3) * 2;
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        const int k = c * D + ks * 16 + kc;
        qf[c][ks][0] = qptr[0] ? *reinterpret_cast<const unsigned*>(qptr[0] + k) : 0u;
        qf[c][ks][1] = qptr[1] ? *reinterpret_cast<const unsigned*>(qptr[1] + k) : 0u;
        qf[c][ks][2] = qptr[0] ? *reinterpret_cast<const unsigned*>(qptr[0] + k + 8) : 0u;
        qf[c][ks][3] = qptr[1] ? *reinterpret_cast<const unsigned*>(qptr[1] + k + 8) : 0u;
      }
  }

  const int last_row = min(row0 + DM_ROWS, n_rows) - 1;
  const int j_hi = prefix + last_row / G;
  const int n_tiles = (seq_len > 0 && j_hi >= 0) ? j_hi / DM_TILE + 1 : 0;
  const int w_first = row0 + rw * 16, w_last = min(w_first + 15, n_rows - 1);
  const int w_pos_lo = prefix + w_first / G, w_pos_hi = (w_first < n_rows) ? prefix + w_last / G : -1;

  // the request's block table, once, in shared memory: no dependent global load per key
  __shared__ int pages_s[DM_PAGES_S];
  const int n_pages = n_tiles > 0 ? j_hi / page + 1 : 0;
  const bool pages_staged = n_pages <= DM_PAGES_S;
  if (pages_staged) {
    for (int i = threadIdx.x; i < n_pages; i += DM_WARPS * 32) pages_s[i] = block_tables[(size_t)b * table_width + i];
    __syncthreads();
  }
  const int page_shift = (page & (page - 1)) == 0 ? 31 - __clz(page) : -1;

  // two threads a key: each brings every other 16-byte piece of the key row and of the value row
  auto load_tile = [&](int tile, int stage) {
    const int key = threadIdx.x >> 1, half = threadIdx.x & 1;
    const int j = tile * DM_TILE + key;
    const bool ok = j <= j_hi;
    size_t slot = 0;
    if (ok) {
      const int lp = page_shift >= 0 ? (j >> page_shift) : (j / page);
      const int pg = pages_staged ? pages_s[lp] : block_tables[(size_t)b * table_width + lp];
      slot = ((size_t)pg * KVH + kvh) * page + (size_t)(j - lp * page);
    }
    unsigned char* ks_ = k_s + stage * K_STAGE;
    unsigned char* vs_ = v_s + stage * V_STAGE;
    const bf16* ksrc = k_cache + slot * DK;
    const bf16* vsrc = v_cache + slot * V;
#pragma unroll
    for (int c = 0; c < CHK / 2; ++c) cp_async_16(ks_ + swz<DK>(key, 2 * c + half), ksrc + (2 * c + half) * 8, ok);
#pragma unroll
    for (int c = 0; c < CHV / 2; ++c) cp_async_16(vs_ + swz<V>(key, 2 * c + half), vsrc + (2 * c + half) * 8, ok);
  };

  float o[2][NT][4];
  float m_run[2][2], l_run[2][2];
#pragma unroll
  for (int c = 0; c < 2; ++c) {
#pragma unroll
    for (int i = 0; i < NT; ++i) o[c][i][0] = o[c][i][1] = o[c][i][2] = o[c][i][3] = 0.f;
    m_run[c][0] = m_run[c][1] = -INFINITY;
    l_run[c][0] = l_run[c][1] = 0.f;
  }
  const float sc = scale * DM_LOG2E;

  const int per_split = (n_tiles + nsplit - 1) / nsplit;
  const int t_begin = nsplit > 1 ? (int)blockIdx.x * per_split : 0;
  const int t_end = nsplit > 1 ? min(n_tiles, t_begin + per_split) : n_tiles;
#pragma unroll
  for (int s = 0; s < DM_STAGES - 1; ++s) {
    if (t_begin + s < t_end) load_tile(t_begin + s, s);
    cp_async_commit();
  }
  for (int t = t_begin; t < t_end; ++t) {
    const int at = t - t_begin;
    if (t + DM_STAGES - 1 < t_end) load_tile(t + DM_STAGES - 1, (at + DM_STAGES - 1) % DM_STAGES);
    cp_async_commit();
    cp_async_wait<DM_STAGES - 1>();
    __syncthreads();
    const unsigned char* ks_ = k_s + (at % DM_STAGES) * K_STAGE;
    const unsigned char* vs_ = v_s + (at % DM_STAGES) * V_STAGE;
    const int j0 = t * DM_TILE;
    if (j0 <= w_pos_hi) {                                    // else the tile lies in these rows' future (warp-uniform)
      const bool need_mask = (j0 + DM_TILE - 1 > w_pos_lo) || (j0 + DM_TILE - 1 > j_hi);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float s_acc[2 * NP][4];
#pragma unroll
        for (int nt = 0; nt < 2 * NP; ++nt) s_acc[nt][0] = s_acc[nt][1] = s_acc[nt][2] = s_acc[nt][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
          for (int np = 0; np < NP; ++np) {
            const int mat = lane >> 3, r = lane & 7;
            const int key = key0 + np * 16 + (mat >> 1) * 8 + r;
            const int ch = c * (D / 8) + ks * 2 + (mat & 1);
            unsigned b0, b1, b2, b3;
            ldmatrix_x4(b0, b1, b2, b3, ks_ + swz<DK>(key, ch));
            mma_bf16(s_acc[2 * np], qf[c][ks], b0, b1);
            mma_bf16(s_acc[2 * np + 1], qf[c][ks], b2, b3);
          }
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 2 * NP; ++nt) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float v = s_acc[nt][e] * sc;
            if (need_mask) {
              const int j = j0 + key0 + nt * 8 + (lane & 3) * 2 + (e & 1);
              v = (j <= pos[e >> 1]) ? v : -INFINITY;
            }
            s_acc[nt][e] = v;
            mx[e >> 1] = fmaxf(mx[e >> 1], v);
          }
        }
        float corr[2], m_use[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
          mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
          const float m_new = fmaxf(m_run[c][r], mx[r]);
          m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;
          corr[r] = exp2f(m_run[c][r] - m_use[r]);
          m_run[c][r] = m_new;
        }
        float rs[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < 2 * NP; ++nt) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float p = exp2f(s_acc[nt][e] - m_use[e >> 1]);
            s_acc[nt][e] = p;
            rs[e >> 1] += p;
          }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
          rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
          l_run[c][r] = l_run[c][r] * corr[r] + rs[r];
        }
#pragma unroll
        for (int i = 0; i < NT; ++i) {
          o[c][i][0] *= corr[0];
          o[c][i][1] *= corr[0];
          o[c][i][2] *= corr[1];
          o[c][i][3] *= corr[1];
        }
#pragma unroll
        for (int kk = 0; kk < NP; ++kk) {
          unsigned pf[4];
          pf[0] = pack_bf16(s_acc[2 * kk][0], s_acc[2 * kk][1]);
          pf[1] = pack_bf16(s_acc[2 * kk][2], s_acc[2 * kk][3]);
          pf[2] = pack_bf16(s_acc[2 * kk + 1][0], s_acc[2 * kk + 1][1]);
          pf[3] = pack_bf16(s_acc[2 * kk + 1][2], s_acc[2 * kk + 1][3]);
#pragma unroll
          for (int i = 0; i < NT; i += 2) {
            const int mat = lane >> 3, r = lane & 7;
            const int key = key0 + kk * 16 + (mat & 1) * 8 + r;
            const int ch = i + (mat >> 1);
            unsigned b0, b1, b2, b3;
            ldmatrix_x4_trans(b0, b1, b2, b3, vs_ + swz<V>(key, ch));
            mma_bf16(o[c][i], pf, b0, b1);
            mma_bf16(o[c][i + 1], pf, b2, b3);
          }
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

  if (split) {
    // warps 1..3 hand their partial results (for the same rows) to warp 0 through the tile buffers
    constexpr int PER = 8 + 8 * NT;
    float* xs = reinterpret_cast<float*>(smem);
    __syncthreads();
    if (warp > 0) {
      float* mine_ = xs + (size_t)(warp - 1) * 32 * PER + lane;
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          mine_[(c * 2 + r) * 32] = m_run[c][r];
          mine_[(4 + c * 2 + r) * 32] = l_run[c][r];
        }
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int i = 0; i < NT; ++i)
#pragma unroll
          for (int e = 0; e < 4; ++e) mine_[(8 + (c * NT + i) * 4 + e) * 32] = o[c][i][e];
    }
    __syncthreads();
    if (warp > 0) return;
    for (int w = 0; w < DM_WARPS - 1; ++w) {
      const float* theirs = xs + (size_t)w * 32 * PER + lane;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float fa[2], fb[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const float ma = m_run[c][r], mb = theirs[(c * 2 + r) * 32];
          const float m_new = fmaxf(ma, mb);
          fa[r] = (ma == -INFINITY) ? 0.f : exp2f(ma - m_new);
          fb[r] = (mb == -INFINITY) ? 0.f : exp2f(mb - m_new);
          l_run[c][r] = l_run[c][r] * fa[r] + theirs[(4 + c * 2 + r) * 32] * fb[r];
          m_run[c][r] = m_new;
        }
#pragma unroll
        for (int i = 0; i < NT; ++i)
#pragma unroll
          for (int e = 0; e < 4; ++e)
            o[c][i][e] = o[c][i][e] * fa[e >> 1] + theirs[(8 + (c * NT + i) * 4 + e) * 32] * fb[e >> 1];
      }
    }
  }

  if (nsplit > 1) {
    // (only warp 0 is left) this block's partial result to scratch; the last block of the (request, kv head) folds
    // all of them in split order
    constexpr int PER = 8 + 8 * NT;
    const size_t group = (size_t)b * KVH + kvh;
    float* mine_ = scratch + (group * max_splits + blockIdx.x) * 32 * PER + lane;
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mine_[(c * 2 + r) * 32] = m_run[c][r];
        mine_[(4 + c * 2 + r) * 32] = l_run[c][r];
      }
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
      for (int i = 0; i < NT; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) mine_[(8 + (c * NT + i) * 4 + e) * 32] = o[c][i][e];
    __threadfence();
    __syncwarp();
    int ticket = 0;
    if (lane == 0) ticket = atomicAdd(&counters[group], 1);
    ticket = __shfl_sync(0xffffffffu, ticket, 0);
    if (ticket != nsplit - 1) return;
    __threadfence();
    if (lane == 0) counters[group] = 0;                      // ready for the next launch
#pragma unroll
    for (int c = 0; c < 2; ++c) {
#pragma unroll
      for (int i = 0; i < NT; ++i) o[c][i][0] = o[c][i][1] = o[c][i][2] = o[c][i][3] = 0.f;
      m_run[c][0] = m_run[c][1] = -INFINITY;
      l_run[c][0] = l_run[c][1] = 0.f;
    }
    for (int w = 0; w < nsplit; ++w) {
      const float* theirs = scratch + (group * max_splits + w) * 32 * PER + lane;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float fa[2], fb[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const float ma = m_run[c][r], mb = __ldcg(theirs + (c * 2 + r) * 32);
          const float m_new = fmaxf(ma, mb);
          fa[r] = (ma == -INFINITY) ? 0.f : exp2f(ma - m_new);
          fb[r] = (mb == -INFINITY) ? 0.f : exp2f(mb - m_new);
          l_run[c][r] = l_run[c][r] * fa[r] + __ldcg(theirs + (4 + c * 2 + r) * 32) * fb[r];
          m_run[c][r] = m_new;
        }
#pragma unroll
        for (int i = 0; i < NT; ++i)
#pragma unroll
          for (int e = 0; e < 4; ++e)
            o[c][i][e] = o[c][i][e] * fa[e >> 1] + __ldcg(theirs + (8 + (c * NT + i) * 4 + e) * 32) * fb[e >> 1];
      }
    }
  }

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const float i1 = l_run[0][r] > 0.f ? 1.f / l_run[0][r] : 0.f;
    const float i2 = l_run[1][r] > 0.f ? 1.f / l_run[1][r] : 0.f;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float v = o[0][i][2 * r + e] * i1 - lambda * (o[1][i][2 * r + e] * i2);
        o[0][i][2 * r + e] = v;
        ss += v * v;
      }
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    const float f = out_scale / sqrtf(ss / (float)V + eps);
    if (optr[r] == nullptr) continue;
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      const int d = i * 8 + (lane & 3) * 2;
      *reinterpret_cast<__nv_bfloat162*>(optr[r] + d) =
          __floats2bfloat162_rn(o[0][i][2 * r] * f, o[0][i][2 * r + 1] * f);
    }
  }
}

template <int D, int V>
int launch_diff_mma(bf16* out, const bf16* proj, int proj_stride, const bf16* k_cache, const bf16* v_cache,
                    const int* block_tables, const int* q_start, const int* seq_lens, int B, int table_width,
                    int max_q_len, int H, int KVH, int page, float scale, float lambda, float eps, float out_scale,
                    float* scratch, int* counters, int max_splits, int kinds, cudaStream_t s) {
  const size_t tiles = (size_t)DM_STAGES * DM_TILE * (2 * D + V) * 2;
  const size_t merge = (size_t)(DM_WARPS - 1) * 32 * (8 + V) * sizeof(float);
  const size_t smem = tiles > merge ? tiles : merge;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_diff_mma_kernel<D, V, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attention_diff_mma_kernel<D, V, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) TS_REFUSE((int)e, "ts_attention_diff_mma: shared memory %zu: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  const int G = H / KVH;
  if (scratch == nullptr || counters == nullptr) max_splits = 1;
  // requests whose rows fit one warp (a single token of up to 16 heads a kv head): the grid's x index is the piece of
  // the keys; the others: it is the row tile.  Each instance leaves the other's requests alone.
  if ((kinds & 1) && G <= 16) {
    ts_launch(attention_diff_mma_kernel<D, V, true>, dim3(max_splits, KVH, B), dim3(DM_WARPS * 32), smem, s, out, proj,
              proj_stride, k_cache, v_cache, block_tables, q_start, seq_lens, table_width, H, KVH, page, scale, lambda, eps,
              out_scale, max_splits > 1 ? scratch : nullptr, counters, max_splits);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) TS_REFUSE((int)e, "ts_attention_diff_mma: %s", cudaGetErrorString(e));
  }
  if ((kinds & 2) && max_q_len * G > 16) {
    ts_launch(attention_diff_mma_kernel<D, V, false>, dim3(ceil_div(max_q_len * G, DM_ROWS), KVH, B), dim3(DM_WARPS * 32), smem,
              s, out, proj, proj_stride, k_cache, v_cache, block_tables, q_start, seq_lens, table_width, H, KVH, page, scale,
              lambda, eps, out_scale, (float*)nullptr, counters, 1);
  }
  TS_LAUNCH_CHECK();
}

}  // namespace

TS_API int ts_attention_diff_mma_supported(int H, int KVH, int D, int V, int dtype) {
  return dtype == TS_BF16 && KVH > 0 && H % KVH == 0 && (D == 32 || D == 64) && (V == 64 || V == 128);
}

// Floats of scratch the kernel wants for `max_splits` pieces of the keys of B requests' single tokens.
TS_API long long ts_attention_diff_mma_scratch_floats(int B, int KVH, int V, int max_splits) {
  return (long long)B * KVH * max_splits * 32 * (8 + V);
}

// Arguments as ts_attention_diff; bfloat16 only; the projection rows and both caches 16-byte aligned.
// scratch / counters (B * KVH ints, zero before the first launch; the kernel leaves them zero) / max_splits: requests
// that bring one token have their keys cut over up to max_splits blocks; null or 1: never.  kinds: bit 0: the step
// has requests whose rows fit one warp, bit 1: it has others (3 when the caller does not know).
TS_API int ts_attention_diff_mma(void* out, const void* proj, int proj_stride, const void* k_cache, const void* v_cache,
                                 const int* block_tables, const int* q_start, const int* seq_lens, int B,
                                 int table_width, int max_q_len, int H, int KVH, int D, int V, int page, float scale,
                                 float lambda, float eps, float out_scale, float* scratch, int* counters,
                                 int max_splits, int kinds, void* stream) {
  if (B <= 0 || max_q_len <= 0) return 0;
  if (!ts_attention_diff_mma_supported(H, KVH, D, V, TS_BF16))
    TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_attention_diff_mma: H=%d KVH=%d D=%d V=%d is not taken by this kernel", H, KVH, D, V);
  if (B > 65535 || KVH > 65535) TS_REFUSE(TS_ERR_LIMIT, "ts_attention_diff_mma: %d requests / %d kv heads", B, KVH);
  if (((uintptr_t)proj | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) & 15 || proj_stride % 8)
    TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_attention_diff_mma: operands must be 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
#define TS_DM(DD, VV)                                                                                                \
  if (D == DD && V == VV)                                                                                            \
    return launch_diff_mma<DD, VV>((bf16*)out, (const bf16*)proj, proj_stride, (const bf16*)k_cache, (const bf16*)v_cache, \
                                   block_tables, q_start, seq_lens, B, table_width, max_q_len, H, KVH, page, scale,   \
                                   lambda, eps, out_scale, scratch, counters, max_splits, kinds, s)
  TS_DM(32, 64);
  TS_DM(32, 128);
  TS_DM(64, 64);
  TS_DM(64, 128);
#undef TS_DM
  TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_attention_diff_mma: no instance");
}
