// Decode kernels: one new token for each of `batch` sequences with ragged lengths.
//   kvm_decode_pre_kernel   per kv row: memory update for sequences whose window start jumps at this
//                           token (one full block leaves the window), direct memory append while the
//                           sequence is shorter than one block, then the ring write of the new token
//   kvm_decode_attn_kernel  split-K joint attention over [memory ; window] with 16-byte loads; the
//                           last split of a kv row combines the partial results, the last kv row of a
//                           sequence advances the sequence's lengths
// Follows model/kvm_mixer.py:572-713 (eager single-token step).
#include "kvm_update.cuh"

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

// Partial result of one split: [m, l, acc[D]] in fp32.
template <int D>
__global__ void __launch_bounds__(kDecThreads)
kvm_decode_attn_kernel(LayerDev L, DecodeCacheDev cache, Tensor4 q, const int* __restrict__ n_append_arr,
                       int rows_per_split, float* __restrict__ partial, int* __restrict__ counters,
                       bf16* __restrict__ out, float sm_scale) {
  constexpr int LPR = D / 8;              // lanes per row (16 bytes each)
  constexpr int RG = kDecThreads / LPR;   // rows in flight per pass
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* sc = reinterpret_cast<float*>(smem_raw);   // [rows_per_split]
  float* red = sc + rows_per_split;                 // [RG][D]
  __shared__ float s_red[kDecThreads / 32];
  __shared__ int s_last;

  const int z = blockIdx.x, nsplit = gridDim.x;
  const int row = blockIdx.y;
  const int b = row / L.Hkv, hkv = row % L.Hkv;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rgi = tid / LPR, li = tid % LPR;
  const int C = L.C, WC = L.W * L.C, G = L.Hq / L.Hkv;
  const int cap = cache.mem.capacity;

  const int past = cache.total_len[b];
  const int n_app = n_append_arr ? n_append_arr[b] : -1;
  int S = cache.state_len[b] + (n_app > 0 ? n_app : 0);
  if (past < C && S == past) S += 1;  // direct append done by the pre kernel
  const int total = past + 1;
  const int new_begin = bswa_begin_dev(total, C, L.W);
  const int S_act = new_begin > 0 ? S : 0;
  const int n_rows = S_act + (total - new_begin);
  const int r_begin = z * rows_per_split;
  const int r_end = min(n_rows, r_begin + rows_per_split);

  const bf16* mk = cache.mem.k_attn + (size_t)row * cap * D;
  const bf16* mv = cache.mem.v_attn + (size_t)row * cap * D;
  const bf16* rk = cache.ring_k + (size_t)row * WC * D;
  const bf16* rv = cache.ring_v + (size_t)row * WC * D;

  auto krow = [&](int r) -> const bf16* {
    return r < S_act ? mk + (size_t)r * D : rk + (size_t)((new_begin + (r - S_act)) % WC) * D;
  };
  auto vrow = [&](int r) -> const bf16* {
    return r < S_act ? mv + (size_t)r * D : rv + (size_t)((new_begin + (r - S_act)) % WC) * D;
  };

  for (int gq = 0; gq < G; ++gq) {
    const int hq = hkv * G + gq;
    const float sc_mem = sm_scale * L.state_temp[hq] * kLog2e;
    const float sc_win = sm_scale * L.front_temp[hq] * kLog2e;
    float qf[8];
    {
      const uint4 u = *reinterpret_cast<const uint4*>(q.row(b, hq, 0) + li * 8);
      float2 a = unpack_bf16(u.x), c = unpack_bf16(u.y), d = unpack_bf16(u.z), e = unpack_bf16(u.w);
      qf[0] = a.x; qf[1] = a.y; qf[2] = c.x; qf[3] = c.y; qf[4] = d.x; qf[5] = d.y; qf[6] = e.x; qf[7] = e.y;
    }
    // pass 1: scores
    float mloc = -INFINITY;
    for (int base = r_begin; base < r_end; base += 4 * RG) {  // trip count uniform over the block
      const int r0 = base + rgi;
      uint4 kv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int r = r0 + u * RG;
        kv[u] = r < r_end ? *reinterpret_cast<const uint4*>(krow(r) + li * 8) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int r = r0 + u * RG;
        float2 a = unpack_bf16(kv[u].x), c = unpack_bf16(kv[u].y), d = unpack_bf16(kv[u].z), e = unpack_bf16(kv[u].w);
        float dot = qf[0] * a.x + qf[1] * a.y + qf[2] * c.x + qf[3] * c.y + qf[4] * d.x + qf[5] * d.y + qf[6] * e.x + qf[7] * e.y;
#pragma unroll
        for (int off = LPR / 2; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
        if (r < r_end) {
          const float x = dot * (r < S_act ? sc_mem : sc_win);
          if (li == 0) sc[r - r_begin] = x;
          mloc = fmaxf(mloc, x);
        }
      }
    }
    mloc = warp_max(mloc);
    if (lane == 0) s_red[warp] = mloc;
    __syncthreads();
    float mblk = s_red[0];
#pragma unroll
    for (int w = 1; w < kDecThreads / 32; ++w) mblk = fmaxf(mblk, s_red[w]);
    const float m_use = mblk == -INFINITY ? 0.f : mblk;
    // pass 2: probabilities and P.V
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float lsum = 0.f;
    for (int base = r_begin; base < r_end; base += 4 * RG) {
      const int r0 = base + rgi;
      uint4 vv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int r = r0 + u * RG;
        vv[u] = r < r_end ? *reinterpret_cast<const uint4*>(vrow(r) + li * 8) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int r = r0 + u * RG;
        if (r < r_end) {
          const float p = exp2f(sc[r - r_begin] - m_use);
          lsum += p;
          float2 a = unpack_bf16(vv[u].x), c = unpack_bf16(vv[u].y), d = unpack_bf16(vv[u].z), e = unpack_bf16(vv[u].w);
          acc[0] += p * a.x; acc[1] += p * a.y; acc[2] += p * c.x; acc[3] += p * c.y;
          acc[4] += p * d.x; acc[5] += p * d.y; acc[6] += p * e.x; acc[7] += p * e.y;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) red[rgi * D + li * 8 + i] = acc[i];
    // every lane of a row group added the same p: keep one copy per row group
    if (li != 0) lsum = 0.f;
    lsum = warp_sum(lsum);
    __syncthreads();  // red[] complete; s_red (max) consumed by everyone
    if (lane == 0) s_red[warp] = lsum;
    __syncthreads();
    float* pout = partial + ((size_t)(b * L.Hq + hq) * nsplit + z) * (D + 2);
    if (tid < D) {
      float a = 0.f;
#pragma unroll 4
      for (int rg = 0; rg < RG; ++rg) a += red[rg * D + tid];
      pout[2 + tid] = a;
    }
    if (tid == 0) {
      float l = 0.f;
#pragma unroll
      for (int w = 0; w < kDecThreads / 32; ++w) l += s_red[w];
      pout[0] = mblk;
      pout[1] = l;
    }
    __syncthreads();
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
  const int nsplit = (max_rows + rows_per_split - 1) / rows_per_split;
  constexpr int RG = kDecThreads / (D / 8);
  const size_t smem_a = (size_t)rows_per_split * 4 + (size_t)RG * D * 4;
  dim3 grid(nsplit > 0 ? nsplit : 1, rows);
  kvm_decode_attn_kernel<D><<<grid, kDecThreads, smem_a, stream>>>(L, cache, q, any_update ? n_append : nullptr,
                                                                  rows_per_split, partial, counters, out,
                                                                  1.0f / sqrtf((float)D));
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
