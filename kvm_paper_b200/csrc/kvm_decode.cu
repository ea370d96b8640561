// Decode kernels: one new token for each of `batch` sequences with ragged lengths.
//   kvm_decode_pre_kernel   per kv row: memory update for sequences whose window start jumps at this
//                           token (one full block leaves the window), direct memory append while the
//                           sequence is shorter than one block, then the ring write of the new token
//   kvm_decode_attn_kernel  split-K joint attention over [memory ; window] with 16-byte loads; the
//                           last split of a kv row combines the partial results, the last kv row of a
//                           sequence advances the sequence's lengths
// Follows model/kvm_mixer.py:572-713 (eager single-token step).
#include "kvm_update.cuh"
#include "kvm_tc.cuh"

namespace kvm {

__device__ __forceinline__ int bswa_begin_dev(int total, int C, int W) {
  const int end = ((total + C - 1) / C) * C;
  return max(0, end - W * C);
}

// ------------------------------------------------------------------------------------------- pre
template <int D, int NT, bool UPDATE, bool SB>
__global__ void __launch_bounds__(NT, 1)
kvm_decode_pre_kernel(LayerDev L, DecodeCacheDev cache, Tensor4 k, Tensor4 v, Tensor4 gate,
                      const int* __restrict__ n_append_arr, bf16* pk_scr, int* route) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int row = blockIdx.x;
  const int b = row / L.Hkv, h = row % L.Hkv;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int C = L.C, WC = L.W * L.C;
  const int past = cache.total_len[b];
  const int S = cache.state_len[b];
  const int cap = cache.mem.capacity;

  MemoryRowPtrs m;
  m.k_sum = cache.mem.k_sum + (size_t)row * cap * D;
  m.v_sum = cache.mem.v_sum + (size_t)row * cap * D;
  m.vlen = cache.mem.vlen + (size_t)row * cap;
  m.k_attn = cache.mem.k_attn + (size_t)row * cap * D;
  m.v_attn = cache.mem.v_attn + (size_t)row * cap * D;
  bf16* rk = cache.ring_k + (size_t)row * WC * D;
  bf16* rv = cache.ring_v + (size_t)row * WC * D;
  bf16* rg = cache.ring_g + (size_t)row * WC;

  if constexpr (UPDATE) {
    const int n_app = n_append_arr ? n_append_arr[b] : -1;
    if (n_app >= 0) {
      // the block [old_begin, old_begin + C) leaves the window (model/kvm_mixer.py:646-669)
      UpdateSmem<D> s;
      s.carve(smem_raw, C, cap, SB);
      const int old_begin = bswa_begin_dev(past, C, L.W);
      const int slot0 = old_begin % WC;
      TokenSrc src;
      src.k = rk + (size_t)slot0 * D; src.k_st = D;
      src.v = rv + (size_t)slot0 * D; src.v_st = D;
      src.g = rg + slot0; src.g_st = 1;
      src.next_k = nullptr; src.next_v = nullptr;
      ViewStore view;  // decode keeps one live copy of the attention view: rows are refreshed in place
      view.k = m.k_attn; view.v = m.v_attn; view.cur = nullptr; view.ver_idx = nullptr; view.pool_next = 0;
      memory_update<D, NT, SB>(L, src, m, view, cap, S, n_app, pk_scr + (size_t)row * C * D,
                               route ? route + (size_t)row * C : nullptr, s);
    }
  }
  // the new token
  if (warp == 0) {
    const bf16* kp = k.row(b, h, 0);
    const bf16* vp = v.row(b, h, 0);
    const bf16 gt = *gate.row(b, h, 0);
    RowVec<D> kr, vr;
    load_row<D>(kr, kp, lane);
    load_row<D>(vr, vp, lane);
    const int slot = past % WC;
    store_row<D>(kr, rk + (size_t)slot * D, lane);
    store_row<D>(vr, rv + (size_t)slot * D, lane);
    if (lane == 0) rg[slot] = gt;
    if (past < C && S == past && past < cap) {
      // still inside the first block: the token becomes memory row `past` directly
      // (model/kvm_mixer.py:623-638; no gating on this path)
      RowVec<D> pk;
      prepare_key_row<D>(L, pk, kp, lane);
      const float vl = row_norm<D>(vr);
      store_row<D>(pk, m.k_sum + (size_t)past * D, lane);
      store_row<D>(vr, m.v_sum + (size_t)past * D, lane);
      if (lane == 0) m.vlen[past] = vl;
      refresh_memory_row<D>(L, pk, vr, vl, m.k_attn + (size_t)past * D, m.v_attn + (size_t)past * D, lane);
    }
  }
}

// ------------------------------------------------------------------------------------- attention
constexpr int kDecThreads = 128;
constexpr int kDecChunk = 128;  // rows per CTA

template <int D>
__host__ __device__ constexpr int dec_row_stride() { return D + 8; }  // padded rows: conflict-free fragment loads

__host__ __device__ inline size_t decode_attn_smem_bytes(int D, int G) {
  return (size_t)2 * kDecChunk * (D + 8) * 2 + (size_t)4 * G * D * 4 + (size_t)2 * 4 * 16 * 4 + 16;
}

// Split-K joint attention of one new token over [memory ; window] on the tensor cores.
// The rows of one kv row form up to three contiguous runs (memory rows, window part up to the end of the
// ring, wrapped window part); CTA z takes one chunk of <= 128 rows of one run.  Every thread pulls one key
// row and one value row into (padded) shared memory with bulk (TMA) copies issued before anything else:
// 64 KB in flight per CTA at no register cost.  All query heads of the kv head (G <= 16) form the M=16
// tile of warp-level MMAs: S = Q K^T (each warp 32 keys), softmax over the chunk, O = P V; one chunk
// costs ~250 warp instructions per warp, so the kernel stays bandwidth-bound.
// Partial result of one chunk and query head: [m, l, acc[D]] in fp32; the last chunk of a kv row combines.
template <int D>
__global__ void __launch_bounds__(kDecThreads)
kvm_decode_attn_kernel(LayerDev L, DecodeCacheDev cache, Tensor4 q, const int* __restrict__ n_append_arr,
                       float* __restrict__ partial, int* __restrict__ counters, bf16* __restrict__ out, float sm_scale,
                       int* __restrict__ status) {
  constexpr int STR = dec_row_stride<D>();
  constexpr int KS = D / 16;   // k-steps of Q K^T
  constexpr int DT8 = D / 8;   // n8 tiles of the output
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int G = L.Hq / L.Hkv;
  bf16* sK = reinterpret_cast<bf16*>(smem_raw);                    // [kDecChunk][STR]
  bf16* sV = sK + (size_t)kDecChunk * STR;                          // [kDecChunk][STR]
  float* ored = reinterpret_cast<float*>(sV + (size_t)kDecChunk * STR);  // [4 warps][G][D]
  float* wmax = ored + (size_t)4 * G * D;                           // [4][16]
  float* wsum = wmax + 64;                                          // [4][16]
  uint64_t* bar = reinterpret_cast<uint64_t*>(wsum + 64);
  __shared__ int s_last;

  const int z = blockIdx.x, nsplit = gridDim.x;
  const int row = blockIdx.y;
  const int b = row / L.Hkv, hkv = row % L.Hkv;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int C = L.C, WC = L.W * L.C;
  const int cap = cache.mem.capacity;

  const int past = cache.total_len[b];
  const int n_app = n_append_arr ? n_append_arr[b] : -1;
  int S = cache.state_len[b] + (n_app > 0 ? n_app : 0);
  if (past < C && S == past) S += 1;  // direct append done by the pre kernel
  const int total = past + 1;
  const int new_begin = bswa_begin_dev(total, C, L.W);
  const int S_act = new_begin > 0 ? S : 0;
  // runs: memory [0,S_act), window part A (ring slots slot0..), window part B (ring slots 0..)
  const int n_win = total - new_begin;
  const int slot0 = new_begin % WC;
  const int len_a = min(n_win, WC - slot0), len_b = n_win - len_a;
  const int c_mem = (S_act + kDecChunk - 1) / kDecChunk, c_a = (len_a + kDecChunk - 1) / kDecChunk;
  const int c_b = (len_b + kDecChunk - 1) / kDecChunk;
  int n = 0;
  bool is_mem = false;
  const bf16* src_k = nullptr;
  const bf16* src_v = nullptr;
  if (z < c_mem) {
    const int r0 = z * kDecChunk;
    n = min(kDecChunk, S_act - r0);
    is_mem = true;
    src_k = cache.mem.k_attn + ((size_t)row * cap + r0) * D;
    src_v = cache.mem.v_attn + ((size_t)row * cap + r0) * D;
  } else if (z < c_mem + c_a) {
    const int r0 = (z - c_mem) * kDecChunk;
    n = min(kDecChunk, len_a - r0);
    src_k = cache.ring_k + ((size_t)row * WC + slot0 + r0) * D;
    src_v = cache.ring_v + ((size_t)row * WC + slot0 + r0) * D;
  } else if (z < c_mem + c_a + c_b) {
    const int r0 = (z - c_mem - c_a) * kDecChunk;
    n = min(kDecChunk, len_b - r0);
    src_k = cache.ring_k + ((size_t)row * WC + r0) * D;
    src_v = cache.ring_v + ((size_t)row * WC + r0) * D;
  }
  if (tid == 0) {
    tc::mbar_init(bar, 1);
    tc::fence_barrier_init();
  }
  __syncthreads();
  if (n > 0) {
    if (tid == 0) tc::mbar_arrive_expect_tx(bar, (uint32_t)(2 * n * D * 2));
    if (tid < n) {  // one key row and one value row per thread
      tc::bulk_g2s(sK + (size_t)tid * STR, src_k + (size_t)tid * D, D * 2, bar);
      tc::bulk_g2s(sV + (size_t)tid * STR, src_v + (size_t)tid * D, D * 2, bar);
    } else {        // rows past the run: zeros (their scores are masked, their values must be finite)
      for (int c = 0; c < D / 8; ++c) {
        *reinterpret_cast<uint4*>(sK + (size_t)tid * STR + c * 8) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(sV + (size_t)tid * STR + c * 8) = make_uint4(0, 0, 0, 0);
      }
    }
  }
  // query fragments of the kv head's G query heads (rows g and g+8 of the M=16 tile), per-row scales
  uint32_t qa[KS][4];
  float scl[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int qh = g + r * 8;
    const bool okq = qh < G;
    const int hq = hkv * G + (okq ? qh : 0);
    scl[r] = sm_scale * (is_mem ? L.state_temp[hq] : L.front_temp[hq]) * kLog2e;
    const bf16* qp = q.row(b, hq, 0) + t * 2;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      qa[ks][r] = okq ? *reinterpret_cast<const uint32_t*>(qp + ks * 16) : 0u;
      qa[ks][2 + r] = okq ? *reinterpret_cast<const uint32_t*>(qp + ks * 16 + 8) : 0u;
    }
  }
  bool ok = true;
  if (n > 0) {
    ok = tc::mbar_wait(bar, 0);
    if (!ok && tid == 0) atomicExch(status, KVM_ERR_DEVICE_TIMEOUT);
  }
  __syncthreads();  // zero-filled rows visible

  float m_row[2] = {-INFINITY, -INFINITY}, l_row[2] = {0.f, 0.f};
  float o[DT8][4];
#pragma unroll
  for (int i = 0; i < DT8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float sacc[4][4];
  if (n > 0 && ok) {
    // S = Q K^T for this warp's 32 keys
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      sacc[j][0] = sacc[j][1] = sacc[j][2] = sacc[j][3] = 0.f;
      const bf16* brow = sK + (size_t)(warp * 32 + j * 8 + g) * STR + t * 2;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(brow + ks * 16);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(brow + ks * 16 + 8);
        mma_bf16_16816(sacc[j], qa[ks], b0, b1);
      }
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = warp * 32 + j * 8 + t * 2 + (e & 1);
        const float x = key < n ? sacc[j][e] * scl[e >> 1] : -INFINITY;
        sacc[j][e] = x;
        mx[e >> 1] = fmaxf(mx[e >> 1], x);
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      if (t == 0) wmax[warp * 16 + g + r * 8] = mx[r];
    }
  } else if (t == 0) {
    wmax[warp * 16 + g] = -INFINITY;
    wmax[warp * 16 + g + 8] = -INFINITY;
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int rr = g + r * 8;
    m_row[r] = fmaxf(fmaxf(wmax[rr], wmax[16 + rr]), fmaxf(wmax[32 + rr], wmax[48 + rr]));
  }
  if (n > 0 && ok) {
    // P = exp2(S - m) and O = P V for this warp's keys
    const float mu0 = m_row[0] == -INFINITY ? 0.f : m_row[0];
    const float mu1 = m_row[1] == -INFINITY ? 0.f : m_row[1];
    uint32_t pa[2][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float p0 = exp2f(sacc[j][0] - mu0), p1 = exp2f(sacc[j][1] - mu0);
      const float p2 = exp2f(sacc[j][2] - mu1), p3 = exp2f(sacc[j][3] - mu1);
      l_row[0] += p0 + p1;
      l_row[1] += p2 + p3;
      pa[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p0, p1);
      pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
      for (int dp = 0; dp < DT8 / 2; ++dp) {
        uint32_t vb[4];
        const bf16* vrow = sV + (size_t)(warp * 32 + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * STR + dp * 16 + (lane >> 4) * 8;
        ldmatrix_x4_trans(vb, vrow);
        mma_bf16_16816(o[dp * 2 + 0], pa[kk], vb[0], vb[1]);
        mma_bf16_16816(o[dp * 2 + 1], pa[kk], vb[2], vb[3]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_row[r] += __shfl_xor_sync(0xffffffffu, l_row[r], 1);
    l_row[r] += __shfl_xor_sync(0xffffffffu, l_row[r], 2);
    if (t == 0) wsum[warp * 16 + g + r * 8] = l_row[r];
  }
  // this warp's partial output rows of the real query heads -> shared memory
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int qh = g + r * 8;
    if (qh < G) {
      float* dst = ored + ((size_t)warp * G + qh) * D + t * 2;
#pragma unroll
      for (int i = 0; i < DT8; ++i) *reinterpret_cast<float2*>(dst + i * 8) = make_float2(o[i][r * 2], o[i][r * 2 + 1]);
    }
  }
  __syncthreads();
  for (int gq = 0; gq < G; ++gq) {
    const int hq = hkv * G + gq;
    float* pout = partial + ((size_t)(b * L.Hq + hq) * nsplit + z) * (D + 2);
    if (tid < D) {
      const float* src = ored + (size_t)gq * D + tid;
      pout[2 + tid] = src[0] + src[(size_t)G * D] + src[(size_t)2 * G * D] + src[(size_t)3 * G * D];
    }
    if (tid == 0) {
      pout[0] = fmaxf(fmaxf(wmax[gq], wmax[16 + gq]), fmaxf(wmax[32 + gq], wmax[48 + gq]));
      pout[1] = wsum[gq] + wsum[16 + gq] + wsum[32 + gq] + wsum[48 + gq];
    }
  }

  // ---- the last split of this kv row combines; the last kv row of the sequence advances lengths
  __threadfence();
  if (tid == 0) {
    const int prev = atomicAdd(&counters[row], 1);
    s_last = (prev == nsplit - 1);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int gq = 0; gq < G; ++gq) {
    const int hq = hkv * G + gq;
    const float* pin = partial + ((size_t)(b * L.Hq + hq) * nsplit) * (D + 2);
    float M = -INFINITY;
    for (int s2 = 0; s2 < nsplit; ++s2) M = fmaxf(M, __ldcg(pin + (size_t)s2 * (D + 2)));
    if (tid < D) {
      float Lsum = 0.f, a = 0.f;
      for (int s2 = 0; s2 < nsplit; ++s2) {
        const float ms = __ldcg(pin + (size_t)s2 * (D + 2));
        const float w = ms == -INFINITY ? 0.f : exp2f(ms - M);
        Lsum += w * __ldcg(pin + (size_t)s2 * (D + 2) + 1);
        a += w * __ldcg(pin + (size_t)s2 * (D + 2) + 2 + tid);
      }
      out[(size_t)b * L.Hq * D + (size_t)hq * D + tid] = __float2bfloat16_rn(Lsum > 0.f ? a / Lsum : 0.f);
    }
  }
  if (tid == 0) {
    counters[row] = 0;
    const int nb = gridDim.y / L.Hkv;
    const int prev = atomicAdd(&counters[nb * L.Hkv + b], 1);
    if (prev == L.Hkv - 1) {
      counters[nb * L.Hkv + b] = 0;
      cache.total_len[b] = total;
      cache.state_len[b] = S;
    }
  }
}

// Rebuild the attention view of rows [0, state_len[b]) from the carried sums.
template <int D>
__global__ void kvm_memory_refresh_kernel(LayerDev L, MemoryDev mem, const int* __restrict__ state_len) {
  const int row = blockIdx.y;
  const int b = row / L.Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + warp;
  if (r >= state_len[b] || r >= mem.capacity) return;
  const size_t off = ((size_t)row * mem.capacity + r) * D;
  RowVec<D> ks, vs;
  load_row<D>(ks, mem.k_sum + off, lane);
  load_row<D>(vs, mem.v_sum + off, lane);
  refresh_memory_row<D>(L, ks, vs, mem.vlen[(size_t)row * mem.capacity + r], mem.k_attn + off, mem.v_attn + off, lane);
}

// ------------------------------------------------------------------------------------- host side
template <int D>
static cudaError_t launch_decode(const LayerDev& L, int batch, const DecodeCacheDev& cache, Tensor4 q, Tensor4 k,
                                 Tensor4 v, Tensor4 gate, const int* n_append, int any_update, int max_rows, bf16* out,
                                 int* route, bf16* pk_scr, bf16* gk_scr, float* partial, int* counters,
                                 int rows_per_split, cudaStream_t stream) {
  constexpr int NT = 512;
  const int rows = batch * L.Hkv;
  cudaError_t e;
  if (any_update) {
    const bool sb = update_block_fits_smem<D>(L.C, cache.mem.capacity);
    const size_t smem_u = UpdateSmem<D>::bytes(L.C, cache.mem.capacity, sb);
    auto kern = sb ? kvm_decode_pre_kernel<D, NT, true, true> : kvm_decode_pre_kernel<D, NT, true, false>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_u);
    if (e != cudaSuccess) return e;
    kern<<<rows, NT, smem_u, stream>>>(L, cache, k, v, gate, n_append, pk_scr, route);
  } else {
    kvm_decode_pre_kernel<D, 32, false, false><<<rows, 32, 0, stream>>>(L, cache, k, v, gate, nullptr, pk_scr, route);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  // up to three runs of rows per kv row (memory, window, wrapped window): two chunks more than the row count needs
  const int nsplit = (max_rows + kDecChunk - 1) / kDecChunk + 2;
  (void)rows_per_split;
  if (L.Hq / L.Hkv > 16) return cudaErrorInvalidValue;  // the query heads of a kv head form one M=16 MMA tile
  const size_t smem_a = decode_attn_smem_bytes(D, L.Hq / L.Hkv);
  e = cudaFuncSetAttribute(kvm_decode_attn_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_a);
  if (e != cudaSuccess) return e;
  dim3 grid(nsplit, rows);
  kvm_decode_attn_kernel<D><<<grid, kDecThreads, smem_a, stream>>>(L, cache, q, any_update ? n_append : nullptr, partial,
                                                                  counters, out, 1.0f / sqrtf((float)D),
                                                                  counters + rows + batch);
  return cudaGetLastError();
}

cudaError_t decode_dispatch(int D, const LayerDev& L, int batch, const DecodeCacheDev& cache, Tensor4 q, Tensor4 k,
                            Tensor4 v, Tensor4 gate, const int* n_append, int any_update, int max_rows, bf16* out,
                            int* route, bf16* pk_scr, bf16* gk_scr, float* partial, int* counters, int rows_per_split,
                            cudaStream_t stream) {
  switch (D) {
    case 32: return launch_decode<32>(L, batch, cache, q, k, v, gate, n_append, any_update, max_rows, out, route, pk_scr, gk_scr, partial, counters, rows_per_split, stream);
    case 64: return launch_decode<64>(L, batch, cache, q, k, v, gate, n_append, any_update, max_rows, out, route, pk_scr, gk_scr, partial, counters, rows_per_split, stream);
    case 128: return launch_decode<128>(L, batch, cache, q, k, v, gate, n_append, any_update, max_rows, out, route, pk_scr, gk_scr, partial, counters, rows_per_split, stream);
  }
  return cudaErrorInvalidValue;
}

cudaError_t refresh_dispatch(int D, const LayerDev& L, int batch, MemoryDev mem, const int* state_len, cudaStream_t stream) {
  dim3 grid((mem.capacity + 7) / 8, batch * L.Hkv);
  switch (D) {
    case 32: kvm_memory_refresh_kernel<32><<<grid, 256, 0, stream>>>(L, mem, state_len); break;
    case 64: kvm_memory_refresh_kernel<64><<<grid, 256, 0, stream>>>(L, mem, state_len); break;
    case 128: kvm_memory_refresh_kernel<128><<<grid, 256, 0, stream>>>(L, mem, state_len); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace kvm
