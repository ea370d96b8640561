// Block attention of the prefill on the Blackwell tensor cores (tcgen05 + tensor memory), head_dim 128.
//
// One CTA = 128 query rows of one (batch, q-head) inside one query block.  Keys/values are consumed in
// tiles of 64 rows: first the memory version of the block (rows gathered from the row pool through the
// version's index table), then the sliding window up to the diagonal.
//
//   warps 4,5   loaders, one per pipeline stage: cp.async of Q and of the K/V tiles into 128B-swizzled
//               operand layouts, fence to the async proxy, mbarrier arrive
//   warp 6      one thread issues tcgen05.mma:  S = Q K^T into tensor memory (two S buffers, so the next
//               score tile is computed while the current one is in softmax), then O += P V
//   warps 0-3   softmax: one query row per thread (= one tensor-memory lane): tcgen05.ld of the score
//               tile, scale by the segment's temperature, mask, exp2, row sum, bf16 P into shared
//               memory for the P V product.  The running maximum is only raised (and O in tensor
//               memory rescaled with tcgen05.ld/st) when a tile exceeds it by more than 2^8, so most
//               tiles need no correction pass.
// Two CTAs fit one SM (112 KB shared memory, 256 tensor-memory columns each): while one CTA is in softmax
// the other one owns the tensor pipe.  Every mbarrier wait is bounded; on expiry the CTA records a
// status code, falls through to the common exit, frees its tensor memory and returns.
#include "kvm_common.cuh"
#include "kvm_tc.cuh"

namespace kvm {

namespace {

constexpr int BM = 128;  // query rows per CTA
constexpr int BN = 64;   // keys per tile
constexpr int HD = 128;  // head dim
constexpr int kThreads = 224;
constexpr int kTmemCols = 256;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

#ifndef KVM_TC_STAGES
#define KVM_TC_STAGES 4
#endif
constexpr int kStages = KVM_TC_STAGES;              // K/V tiles in flight per CTA
constexpr int kCtasPerSm = kStages <= 2 ? 2 : 1;
constexpr uint32_t kOffQ = 0;                       // 2 x [128][64] bf16
constexpr uint32_t kOffK = 32768;                   // kStages x 2 x [64][64]
constexpr uint32_t kOffV = kOffK + kStages * 16384; // kStages x 2 x [64 keys][64]
constexpr uint32_t kOffP = kOffV + kStages * 16384; // [128][64]
constexpr uint32_t kOffBar = kOffP + 16384;         // barriers and scalars
constexpr uint32_t kSmemBytes = kOffBar + 128;

struct Bars {
  uint64_t q_full, kv_full[kStages], kv_empty[kStages], s_full[2], p_full, pv_done;
  uint32_t tmem_base;
  uint32_t abort_flag;
};

// All 32 lanes wait; the result is made uniform over the warp so that no lane leaves a loop alone.
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity) {
  const bool ok = tc::mbar_wait(bar, parity);
  return __all_sync(0xffffffffu, ok);
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

}  // namespace

__global__ void __launch_bounds__(kThreads, kCtasPerSm)
kvm_attn_prefill_tc_kernel(LayerDev L, long long T, Tensor4 q, Tensor4 k, Tensor4 v,
                           const kvm_update_plan* __restrict__ plan, const bf16* __restrict__ pool_k,
                           const bf16* __restrict__ pool_v, long long pool_rows, const int* __restrict__ ver_idx,
                           long long ver_rows, bf16* __restrict__ out, int tiles_per_block, float sm_scale,
                           int* __restrict__ status) {
  extern __shared__ __align__(1024) unsigned char smem[];
  Bars* bars = reinterpret_cast<Bars*>(smem + kOffBar);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int C = L.C;

  const int xi = gridDim.x - 1 - blockIdx.x;  // later (heavier) tiles first
  const int j = xi / tiles_per_block;
  const int ti = xi % tiles_per_block;
  const int qrow = blockIdx.y;
  const int b = qrow / L.Hq, hq = qrow % L.Hq;
  const int hkv = hq / (L.Hq / L.Hkv);
  const long long q0 = (long long)j * C + (long long)ti * BM;
  const long long q_blk_end = min(T, (long long)(j + 1) * C);
  if (q0 >= q_blk_end) return;
  const long long q_tile_end = min(q_blk_end, q0 + BM);
  if ((tc::smem_u32(smem) & 1023u) != 0) {  // operand tiles need 1024-byte alignment
    if (tid == 0) atomicExch(status, KVM_ERR_UNSUPPORTED);
    return;
  }

  int S = 0;
  const bf16* mk = nullptr;
  const bf16* mv = nullptr;
  const int* midx = nullptr;
  if (j >= L.W) {
    const kvm_update_plan pl = plan[j - L.W];
    S = pl.state_before + pl.n_append;
    const size_t kvrow = (size_t)(b * L.Hkv + hkv);
    mk = pool_k + kvrow * pool_rows * HD;
    mv = pool_v + kvrow * pool_rows * HD;
    midx = ver_idx + kvrow * ver_rows + pl.version_row;
  }
  const long long bb = max(0LL, (long long)(j + 1 - L.W) * C);
  const int n_mem_tiles = (S + BN - 1) / BN;
  const int n_win_tiles = (int)((q_tile_end - bb + BN - 1) / BN);
  const int n_tiles = n_mem_tiles + n_win_tiles;

  if (tid == 0) {
    tc::mbar_init(&bars->q_full, 1);
    for (int i = 0; i < kStages; ++i) {
      tc::mbar_init(&bars->kv_full[i], 1);
      tc::mbar_init(&bars->kv_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) tc::mbar_init(&bars->s_full[i], 1);
    tc::mbar_init(&bars->p_full, 4);
    tc::mbar_init(&bars->pv_done, 1);
    bars->abort_flag = 0;
    tc::fence_barrier_init();
  }
  if (warp == 6) tc::tmem_alloc(&bars->tmem_base, kTmemCols);
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem = bars->tmem_base;
  const uint32_t sQ = tc::smem_u32(smem + kOffQ), sK = tc::smem_u32(smem + kOffK);
  const uint32_t sV = tc::smem_u32(smem + kOffV), sP = tc::smem_u32(smem + kOffP);
  bool failed = false;

  if (warp == 4 || warp == 5) {
    // ------------------------------------------------------------------ loaders (warp 4: even tiles + Q, warp 5: odd tiles)
    const int lw = warp - 4;  // this loader takes the tiles t with t % 2 == lw
    const bf16* kbase = k.row(b, hkv, 0);
    const bf16* vbase = v.row(b, hkv, 0);
    if (lw == 0) {
      for (int c = lane; c < BM * 16; c += 32) {
        const int r = c >> 4, cc = c & 15;
        const long long row = q0 + r;
        const bool ok = row < q_tile_end;
        const bf16* src = q.row(b, hq, ok ? row : q0) + cc * 8;
        cp_async16(smem + kOffQ + (cc >> 3) * 16384 + tc::sw128_offset(r, (cc & 7) * 8), src, ok ? 16 : 0);
      }
    }
    for (int t = lw; t < n_tiles; t += 2) {
      const int stage = t % kStages;
      unsigned char* dK = smem + kOffK + stage * 16384;
      unsigned char* dV = smem + kOffV + stage * 16384;
      if (t >= kStages && !warp_wait(&bars->kv_empty[stage], ((t / kStages) - 1) & 1)) { failed = true; break; }
      // lane -> fixed 16-byte column chunk cc and row parity; iteration `it` covers rows 2*it and 2*it+1
      const int cc = lane & 15, rh = lane >> 4;
      const uint32_t col_off = (uint32_t)(cc >> 3) * 8192u;
      if (t < n_mem_tiles) {
        const int row0 = t * BN;
        const int i0 = row0 + lane < S ? __ldg(midx + row0 + lane) : 0;
        const int i1 = row0 + 32 + lane < S ? __ldg(midx + row0 + 32 + lane) : 0;
#pragma unroll
        for (int it = 0; it < BN / 2; ++it) {
          const int r = it * 2 + rh;
          const int a0 = __shfl_sync(0xffffffffu, it < 16 ? i0 : i1, r & 31);
          const bool ok = row0 + r < S;
          const uint32_t off = col_off + (uint32_t)(r * 128) + (uint32_t)((((cc & 7) ^ (r & 7)) & 7) << 4);
          const size_t src = (size_t)a0 * HD + cc * 8;
          cp_async16(dK + off, mk + src, ok ? 16 : 0);
          cp_async16(dV + off, mv + src, ok ? 16 : 0);
        }
      } else {
        const long long r0 = bb + (long long)(t - n_mem_tiles) * BN;
        const bf16* pk = kbase + (r0 + rh) * k.st + cc * 8;
        const bf16* pv = vbase + (r0 + rh) * v.st + cc * 8;
        const int n_ok = (int)min((long long)BN, q_tile_end - r0);  // rows of this tile that exist
#pragma unroll
        for (int it = 0; it < BN / 2; ++it) {
          const int r = it * 2 + rh;
          const bool ok = r < n_ok;
          const uint32_t off = col_off + (uint32_t)(r * 128) + (uint32_t)((((cc & 7) ^ (r & 7)) & 7) << 4);
          cp_async16(dK + off, ok ? pk + (long long)it * 2 * k.st : kbase, ok ? 16 : 0);
          cp_async16(dV + off, ok ? pv + (long long)it * 2 * v.st : vbase, ok ? 16 : 0);
        }
      }
      cp_async_commit();
      cp_async_wait<0>();       // this warp's tile (and Q, the first time) has landed
      tc::fence_proxy_async();  // generic-proxy writes -> visible to the tensor core's operand reads
      __syncwarp();
      if (lane == 0) {
        if (t == 0) tc::mbar_arrive(&bars->q_full);
        tc::mbar_arrive(&bars->kv_full[stage]);
      }
    }
    cp_async_wait<0>();
  } else if (warp == 6) {
    // ------------------------------------------------------------------ MMA issue (one thread)
    if (lane == 0) {
      constexpr uint32_t idesc_qk = tc::make_idesc(BM, BN, 0, 0);
      constexpr uint32_t idesc_pv = tc::make_idesc(BM, HD, 0, 1);
      auto issue_qk = [&](int t) {
        const int stage = t % kStages, sbuf = t & 1;
        const uint32_t d = tmem + (uint32_t)(sbuf * BN);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint64_t da = tc::make_desc(sQ + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024);
          const uint64_t db = tc::make_desc(sK + stage * 16384 + (ks >> 2) * 8192 + (ks & 3) * 32, 16, 1024);
          tc::mma_ss(d, da, db, idesc_qk, ks > 0);
        }
        tc::mma_commit(&bars->s_full[sbuf]);
      };
      if (!tc::mbar_wait(&bars->q_full, 0)) failed = true;
      for (int t = 0; t < 2 && t < n_tiles && !failed; ++t) {
        if (!tc::mbar_wait(&bars->kv_full[t % kStages], 0)) { failed = true; break; }
        tc::tc_fence_after_sync();
        issue_qk(t);
      }
      for (int t = 0; t < n_tiles && !failed; ++t) {
        if (!tc::mbar_wait(&bars->p_full, t & 1)) { failed = true; break; }
        tc::tc_fence_after_sync();
        const int stage = t % kStages;
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks) {
          const uint64_t da = tc::make_desc(sP + ks * 32, 16, 1024);
          const uint64_t db = tc::make_desc(sV + stage * 16384 + ks * 2048, 8192, 1024);
          tc::mma_ss(tmem + 128, da, db, idesc_pv, (t > 0) || (ks > 0));
        }
        tc::mma_commit(&bars->kv_empty[stage]);
        tc::mma_commit(&bars->pv_done);
        if (t + 2 < n_tiles) {
          if (!tc::mbar_wait(&bars->kv_full[(t + 2) % kStages], ((t + 2) / kStages) & 1)) { failed = true; break; }
          tc::tc_fence_after_sync();
          issue_qk(t + 2);
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ softmax (one query row per thread)
    const int row = tid;  // 0..127 == tensor-memory lane
    const long long qpos = q0 + row;
    const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
    const float scale_mem = sm_scale * L.state_temp[hq] * kLog2e;
    const float scale_win = sm_scale * L.front_temp[hq] * kLog2e;
    float m_run = -INFINITY, l_run = 0.f;
    unsigned char* prow = smem + kOffP + row * 128;
    for (int t = 0; t < n_tiles && !failed; ++t) {
      const int stage = t & 1;
      if (!warp_wait(&bars->s_full[stage], (t >> 1) & 1)) { failed = true; break; }
      tc::tc_fence_after_sync();
      uint32_t sr[2][32];
      tc::tmem_ld32(lane_addr + (uint32_t)(stage * BN), sr[0]);
      tc::tmem_ld32(lane_addr + (uint32_t)(stage * BN + 32), sr[1]);
      tc::tmem_ld_wait();
      const bool is_mem = t < n_mem_tiles;
      const long long base = is_mem ? (long long)t * BN : bb + (long long)(t - n_mem_tiles) * BN;
      const float sc = is_mem ? scale_mem : scale_win;
      // keys [0, n_ok) of this tile are visible to this row (memory: rows below S; window: causal)
      const int n_ok = (int)max(0LL, min((long long)BN, (is_mem ? (long long)S : qpos + 1) - base));
      const bool tile_masked = is_mem ? (base + BN > S) : (base + BN > q0 + 1);  // uniform over the CTA
      if (tile_masked) {
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (i >= n_ok) sr[i >> 5][i & 31] = 0xff800000u;  // -inf
      }
      float tm0 = -INFINITY, tm1 = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        tm0 = fmaxf(tm0, __uint_as_float(sr[0][i]));
        tm1 = fmaxf(tm1, __uint_as_float(sr[1][i]));
      }
      const float tmax = fmaxf(tm0, tm1) * sc;  // sc > 0
      const bool need = tmax > m_run + kRescaleThreshold || (m_run == -INFINITY && tmax > -INFINITY);
      const bool warp_need = __any_sync(0xffffffffu, need);
      if (t > 0 && !warp_wait(&bars->pv_done, (t - 1) & 1)) { failed = true; break; }
      if (warp_need) {
        const float m_new = fmaxf(m_run, tmax);
        const float alpha = (m_run == -INFINITY) ? 0.f : ex2(m_run - m_new);
        l_run *= alpha;
        if (t > 0) {  // rescale the running output of this warp's 32 rows in tensor memory
          tc::tc_fence_after_sync();
#pragma unroll
          for (int cb = 0; cb < HD / 32; ++cb) {
            uint32_t o[32];
            tc::tmem_ld32(lane_addr + 128 + cb * 32, o);
            tc::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tc::tmem_st32(lane_addr + 128 + cb * 32, o);
          }
          tc::tmem_st_wait();
        }
        m_run = m_new;
      }
      const float neg_m = (m_run == -INFINITY) ? 0.f : -m_run;
      float ls0 = 0.f, ls1 = 0.f;
#pragma unroll
      for (int cchunk = 0; cchunk < 8; ++cchunk) {
        uint32_t pk[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = cchunk * 8 + e * 2;
          const float p0 = ex2(fmaf(__uint_as_float(sr[i >> 5][i & 31]), sc, neg_m));
          const float p1 = ex2(fmaf(__uint_as_float(sr[(i + 1) >> 5][(i + 1) & 31]), sc, neg_m));
          ls0 += p0;
          ls1 += p1;
          pk[e] = pack_bf16(p0, p1);
        }
        *reinterpret_cast<uint4*>(prow + (((cchunk ^ (row & 7)) & 7) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
      const float ls = ls0 + ls1;
      l_run += ls;
      tc::fence_proxy_async();
      tc::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&bars->p_full);
    }
    // epilogue: O / l -> bf16 -> [B, T, Hq*D]
    if (!failed && !warp_wait(&bars->pv_done, (n_tiles - 1) & 1)) failed = true;
    if (!failed) {
      tc::tc_fence_after_sync();
      const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
      bf16* orow = out + ((long long)b * T + qpos) * ((long long)L.Hq * HD) + (long long)hq * HD;
#pragma unroll
      for (int cb = 0; cb < HD / 32; ++cb) {
        uint32_t o[32];
        tc::tmem_ld32(lane_addr + 128 + cb * 32, o);
        tc::tmem_ld_wait();
        if (qpos < q_tile_end) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 w;
            w.x = pack_bf16(__uint_as_float(o[i * 8 + 0]) * inv, __uint_as_float(o[i * 8 + 1]) * inv);
            w.y = pack_bf16(__uint_as_float(o[i * 8 + 2]) * inv, __uint_as_float(o[i * 8 + 3]) * inv);
            w.z = pack_bf16(__uint_as_float(o[i * 8 + 4]) * inv, __uint_as_float(o[i * 8 + 5]) * inv);
            w.w = pack_bf16(__uint_as_float(o[i * 8 + 6]) * inv, __uint_as_float(o[i * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + cb * 32 + i * 8) = w;
          }
        }
      }
    }
  }
  if (failed) atomicExch(status, KVM_ERR_DEVICE_TIMEOUT);
  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == 6) tc::tmem_dealloc(tmem, kTmemCols);
}

cudaError_t launch_attn_tc(const LayerDev& L, int batch, long long T, Tensor4 q, Tensor4 k, Tensor4 v,
                           const kvm_update_plan* plan_dev, const bf16* pool_k, const bf16* pool_v, long long pool_rows,
                           const int* ver_idx, long long ver_rows, bf16* out, int* status, cudaStream_t stream) {
  const int n_qblocks = (int)((T + L.C - 1) / L.C);
  const int tiles_per_block = L.C / BM;
  cudaError_t e = cudaFuncSetAttribute(kvm_attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
  if (e != cudaSuccess) return e;
  dim3 grid(n_qblocks * tiles_per_block, batch * L.Hq);
  kvm_attn_prefill_tc_kernel<<<grid, kThreads, kSmemBytes, stream>>>(L, T, q, k, v, plan_dev, pool_k, pool_v, pool_rows, ver_idx,
                                                                    ver_rows, out, tiles_per_block, 1.0f / sqrtf((float)HD),
                                                                    status);
  return cudaGetLastError();
}

}  // namespace kvm
