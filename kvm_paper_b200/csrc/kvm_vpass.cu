// The VALUE side of the memory chain (head_dim 128, blocks of 128 / 256 tokens), which no later update reads and
// which therefore runs behind the routing kernel, fully parallel:
//
//   kvm_vdelta_kernel   one job per (kv row, update): delta[touched rows x D] = onehot[rows x tokens] x gv[tokens x D]
//                       on the tensor cores, gv = bf16(v * gate) formed in shared memory from the block's values
//                       (tiled TMA), the touched rows compacted onto the 128 accumulator lanes exactly as the routing
//                       kernel compacted them; bf16(delta) goes to the pool row the version table names for
//                       (update, row) -- as an intermediate that the second kernel replaces --, and one bit per
//                       memory row says whether the update touched it.  The jobs are independent: persistent CTAs
//                       take them in turn, the next job's values are in flight while the current one is finished.
//   kvm_vapply_kernel   one warp per memory row walks the updates that touched its row (the bit table), in order:
//                       row = bf16(row + delta), value view = normalize(row) * magnitude written over the delta.
//                       This is the only sequential part (one bf16 rounding per update and row), a few loads and
//                       stores per touched update.
// Follows model/kvm_mixer.py:231-248 (appended rows) and :321-340 (merged values); products of the one-hot
// contraction are exact, its accumulation order is the hardware's and fixed.
#include <algorithm>

#include "kvm_common.cuh"
#include "kvm_tc.cuh"
#include "kvm_tma_host.cuh"

namespace kvm {
namespace vside {

constexpr int HD = 128;
constexpr int kThreads = 512;
constexpr uint32_t kTmemCols = 256;   // two accumulators of 128 rows x 128 columns

__host__ __device__ inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

struct Layout {
  uint32_t V, O, gs, idx, rows, tl, bars, total;
  __host__ __device__ Layout(int C, int s_max) {
    const uint32_t sp = (uint32_t)((s_max + 63) & ~31);
    uint32_t off = 0;
    V = off;    off += (uint32_t)C * 256u;       // the block's values, then gated: [2 halves of D][C][64], 128-byte swizzle
    O = off;    off += 2u * (uint32_t)C * 256u;  // two one-hot operands [C/64][128 rows][64 tokens]: touched rows 0..127 and 128..255
    gs = off;   off += (uint32_t)C * 4u;         // gates (fp32)
    idx = off;  off += (uint32_t)C * 4u;         // merge target of every token (-1: appended)
    rows = off; off += sp * 4u;                  // stamps[sp] u16 (job that last touched the row), gci[sp] i16
    tl = off;   off += (uint32_t)C * 2u;         // touched rows by compact index
    bars = off; off += 128u;
    total = (off + 15u) & ~15u;
  }
};

struct Bars {
  uint64_t full_v, mma_done;
  uint32_t tmem_base;
  int abort;
  int red[16];
};

struct Maps {
  CUtensorMap v;     // the values [B, H, T, D] (dimensions ordered by stride), boxes of 64 elements x C tokens
  int head_inner;
};

__device__ __forceinline__ bool wait(uint64_t* bar, uint32_t parity, uint32_t limit) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (tc::mbar_try_wait(bar, parity)) return true;
    if (i >= 4096) __nanosleep(100);
  }
  return false;
}

__global__ void __launch_bounds__(kThreads, 1)
kvm_vdelta_kernel(LayerDev L, Tensor4 gate, const kvm_update_plan* __restrict__ plan, int n_plan, int rows,
                  const int* __restrict__ route, bf16* __restrict__ pool_v, long long pool_rows,
                  const int* __restrict__ ver_idx, long long ver_rows, unsigned* __restrict__ tbits, int words, int s_max,
                  int* __restrict__ status, uint32_t wait_limit, const __grid_constant__ Maps maps) {
  extern __shared__ __align__(1024) unsigned char smem[];
  if (*status != 0) return;  // the routing kernel gave up: its decisions and version tables are not to be trusted
  const int C = L.C;
  const Layout lay(C, s_max);
  Bars* bars = reinterpret_cast<Bars*>(smem + lay.bars);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  float* gs = reinterpret_cast<float*>(smem + lay.gs);
  int* idx = reinterpret_cast<int*>(smem + lay.idx);
  unsigned short* stamps = reinterpret_cast<unsigned short*>(smem + lay.rows);
  short* gci = reinterpret_cast<short*>(smem + lay.rows) + ((s_max + 63) & ~31);
  unsigned short* tl = reinterpret_cast<unsigned short*>(smem + lay.tl);
  if (tid == 0) {
    tc::mbar_init(&bars->full_v, 1);
    tc::mbar_init(&bars->mma_done, 1);
    bars->abort = 0;
    tc::fence_barrier_init();
  }
  for (int i = tid; i < s_max; i += kThreads) stamps[i] = 0;
  if (warp == 0) tc::tmem_alloc(&bars->tmem_base, kTmemCols);
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem = bars->tmem_base;
  const int n_jobs = rows * (n_plan - 1);
  uint32_t n_v = 0, n_mma = 0;  // uses of the two barriers so far
  bool ok = true;

  // job j: kv row j % rows, update 1 + j / rows (neighbouring CTAs read neighbouring rows of the same block)
  auto load_values = [&](int j) {  // one thread
    const int row = j % rows, u = 1 + j / rows;
    const int b = row / L.Hkv, h = row % L.Hkv;
    tc::mbar_arrive_expect_tx(&bars->full_v, (uint32_t)C * 256u);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      void* dst = smem + lay.V + half * C * 128;
      if (maps.head_inner) tc::tma_load_4d(dst, &maps.v, half * 64, h, u * C, b, &bars->full_v);
      else tc::tma_load_4d(dst, &maps.v, half * 64, u * C, h, b, &bars->full_v);
    }
  };
  auto has_merges = [&](int j) { return plan[1 + j / rows].n_append < C; };
  auto load_next = [&](int j) {  // one thread, once the current job no longer reads the value buffer
    const int nj = j + gridDim.x;
    if (nj < n_jobs && has_merges(nj)) load_values(nj);
  };

  int job = blockIdx.x;
  if (tid == 0 && job < n_jobs && has_merges(job)) load_values(job);
  // the routing decision and the gate of this thread's token of a job (requested one job ahead)
  auto fetch = [&](int j, int& dec, float& g) {
    dec = -1;
    g = 0.f;
    if (j < n_jobs && tid < C) {
      const int row = j % rows, u = 1 + j / rows;
      dec = route[((size_t)row * n_plan + u) * C + tid];
      g = __bfloat162float(*gate.row(row / L.Hkv, row % L.Hkv, (long long)u * C + tid));
    }
  };
  int my_next;
  float g_next;
  fetch(job, my_next, g_next);
  for (; job < n_jobs && ok; job += gridDim.x) {
    const int row = job % rows, u = 1 + job / rows;
    const kvm_update_plan pl = plan[u];
    const int S1 = pl.state_before + pl.n_append;
    const bool merges = pl.n_append < C;
    const unsigned short stamp = (unsigned short)(1 + (job / (int)gridDim.x));  // unique per job of this CTA
    // ---- routing decisions and gates of the block; touched rows and their compact order
    const int my = my_next;
    if (tid < C) {
      gs[tid] = g_next;
      if (my >= 0) stamps[my] = stamp;
    }
    fetch(job + gridDim.x, my_next, g_next);
    __syncthreads();
    int n_touched = 0;
    for (int r0 = 0; r0 < words * 32; r0 += kThreads) {
      const int r = r0 + tid;
      const bool t = r < S1 && stamps[r] == stamp;
      const unsigned bal = __ballot_sync(0xffffffffu, t);
      if (lane == 0) {
        bars->red[warp] = __popc(bal);
        if ((r >> 5) < words) tbits[((size_t)row * n_plan + u) * words + (r >> 5)] = bal;
      }
      __syncthreads();
      int cnt = bars->red[lane & 15];
#pragma unroll
      for (int d = 1; d < 16; d <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, cnt, d, 16);
        if ((lane & 15) >= d) cnt += y;
      }
      const int total = __shfl_sync(0xffffffffu, cnt, 15);
      const int before = __shfl_sync(0xffffffffu, cnt, max(warp - 1, 0));
      if (t) {
        const int gi = n_touched + (warp > 0 ? before : 0) + __popc(bal & ((1u << lane) - 1u));
        gci[r] = (short)gi;
        tl[gi] = (unsigned short)r;
      }
      n_touched += total;
      __syncthreads();
    }
    if (!merges) {  // nothing was merged in this update (whole block appended): only the bit table
      if (tid == 0) load_next(job);
      continue;
    }
    // ---- one-hot operands: touched row with compact index c in tile c / 128, accumulator lane c % 128
    const int n_tiles = ceil_div(n_touched, 128);  // 1 or 2 (at most C - 1 rows are touched)
    {
      uint4* o = reinterpret_cast<uint4*>(smem + lay.O);
      for (int i = tid; i < n_tiles * C * 16; i += kThreads) o[i] = make_uint4(0, 0, 0, 0);
    }
    // ---- gv = bf16(v * gate) in place (the swizzle permutes 16-byte pieces inside a row: piece i belongs to token (i % 8C) / 8)
    ok = wait(&bars->full_v, n_v & 1, wait_limit);
    ++n_v;
    if (L.gate_values) {
      uint4* v4 = reinterpret_cast<uint4*>(smem + lay.V);
      for (int i = tid; i < C * 16; i += kThreads) {
        const __nv_bfloat162 g2 = __float2bfloat162_rn(gs[(i % (C * 8)) >> 3]);
        uint4 x = v4[i];
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&x);
#pragma unroll
        for (int e = 0; e < 4; ++e) h2[e] = __hmul2(h2[e], g2);
        v4[i] = x;
      }
    }
    __syncthreads();
    if (my >= 0) {
      const int c = gci[my];
      *reinterpret_cast<unsigned short*>(smem + lay.O + (uint32_t)(c >> 7) * (uint32_t)(C * 256) + (uint32_t)(tid >> 6) * (128u * 128u) +
                                         tc::sw128_offset(c & 127, tid & 63)) = 0x3F80;  // bf16 1.0
    }
    // this thread's share of the result: per tile, row = lane quarter * 32 + lane, 32 of its 128 elements; its pool rows
    const int quarter = warp & 3, colq = warp >> 2;
    const int ci = quarter * 32 + lane;
    int slot[2];
#pragma unroll
    for (int t = 0; t < 2; ++t)
      slot[t] = t * 128 + ci < n_touched ? ver_idx[(size_t)row * ver_rows + pl.version_row + tl[t * 128 + ci]] : -1;
    tc::fence_proxy_async();  // the gated values and the one-hot rows -> visible to the tensor core
    tc::tc_fence_before_sync();
    __syncthreads();
    if (tid == 0) {
      tc::tc_fence_after_sync();
      constexpr uint32_t idesc = tc::make_idesc(128, HD, 0, 1);
      const uint64_t db0 = tc::make_desc(tc::smem_u32(smem + lay.V), (uint32_t)C * 128u, 1024);
      for (int t = 0; t < n_tiles; ++t) {
        const uint64_t da0 = tc::make_desc(tc::smem_u32(smem + lay.O + t * C * 256), 16, 1024);
        for (int ks = 0; ks < C / 16; ++ks) {
          const uint64_t da = da0 + (uint64_t)(((uint32_t)(ks >> 2) * (128u * 128u) + (uint32_t)(ks & 3) * 32u) >> 4);
          const uint64_t db = db0 + (uint64_t)(((uint32_t)ks * 2048u) >> 4);
          tc::mma_ss(tmem + (uint32_t)(t * 128), da, db, idesc, ks > 0);
        }
      }
      tc::mma_commit(&bars->mma_done);
    }
    ok = ok && wait(&bars->mma_done, n_mma & 1, wait_limit);
    ++n_mma;
    if (tid == 0) load_next(job);  // the values are consumed: the next job's block may land
    tc::tc_fence_after_sync();
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      if (t < n_tiles) {
        uint32_t d[32];
        tc::tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(t * 128 + colq * 32), d);
        tc::tmem_ld_wait();
        if (slot[t] >= 0) {
          bf16* dst = pool_v + ((size_t)row * pool_rows + slot[t]) * HD + colq * 32;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o4;
            o4.x = pack_bf16(__uint_as_float(d[j * 8 + 0]), __uint_as_float(d[j * 8 + 1]));
            o4.y = pack_bf16(__uint_as_float(d[j * 8 + 2]), __uint_as_float(d[j * 8 + 3]));
            o4.z = pack_bf16(__uint_as_float(d[j * 8 + 4]), __uint_as_float(d[j * 8 + 5]));
            o4.w = pack_bf16(__uint_as_float(d[j * 8 + 6]), __uint_as_float(d[j * 8 + 7]));
            *reinterpret_cast<uint4*>(dst + j * 8) = o4;
          }
        }
      }
    }
    tc::tc_fence_before_sync();
    ok = __syncthreads_and(ok ? 1 : 0) != 0;  // the accumulators and the one-hot buffers are free again
  }
  if (!ok && tid == 0) atomicExch(status, KVM_ERR_DEVICE_TIMEOUT);
  if (!ok) {
    for (int k2 = 0; k2 < 64; ++k2) __nanosleep(1000);  // a copy of this CTA may still be in flight
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, kTmemCols);
}

// ------------------------------------------------------------------------------------------------ apply
constexpr int kApWarps = 8;

// One warp per memory row.  born[row * s_final + r]: the token that created memory row r.
__global__ void __launch_bounds__(kApWarps * 32, 4)
kvm_vapply_kernel(LayerDev L, Tensor4 v, Tensor4 gate, const kvm_update_plan* __restrict__ plan, int n_plan,
                  const int* __restrict__ born, MemoryDev mem, bf16* __restrict__ pool_v, long long pool_rows,
                  const int* __restrict__ ver_idx, long long ver_rows, const unsigned* __restrict__ tbits, int words,
                  int s_final, const int* __restrict__ status) {
  if (*status != 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.y;
  const int b = row / L.Hkv, h = row % L.Hkv;
  const int r = blockIdx.x * kApWarps + warp;
  if (r >= s_final) return;
  const int C = L.C, log2c = C == 256 ? 8 : 7;
  const bool versions = pool_v != nullptr && ver_idx != nullptr;
  // ---- the row is born from one token: value (gated where the layer says so) and magnitude
  const int t_b = born[(size_t)row * s_final + r];
  const int u_b = t_b >> log2c;
  float x[4], vl;
  {
    const uint2 raw = *reinterpret_cast<const uint2*>(v.row(b, h, t_b) + lane * 4);
    const float g = __bfloat162float(*gate.row(b, h, t_b));
    const float2 p0 = unpack_bf16(raw.x), p1 = unpack_bf16(raw.y);
    float o[4] = {p0.x, p0.y, p1.x, p1.y};
    const bool gated = u_b == 0 ? (L.gate_initial != 0) : (L.gate_appends != 0 && L.gate_values != 0);
    if (u_b > 0 && gated) {
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = bf16_round(o[e] * g);
    }
    vl = sqrtf(warp_sum(o[0] * o[0] + o[1] * o[1] + o[2] * o[2] + o[3] * o[3]));  // initial rows: of the ungated value
#pragma unroll
    for (int e = 0; e < 4; ++e) x[e] = (u_b == 0 && gated) ? bf16_round(o[e] * g) : o[e];
  }
  auto view = [&](uint2& o) {  // normalize(row) * magnitude
    const float nrm = fmaxf(sqrtf(warp_sum(x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3])), 1e-12f);
    float y[4] = {x[0], x[1], x[2], x[3]};
    divide_by(y, nrm);
    o.x = pack_bf16(y[0] * vl, y[1] * vl);
    o.y = pack_bf16(y[2] * vl, y[3] * vl);
  };
  const unsigned* bits = tbits + (size_t)row * n_plan * words + (r >> 5);
  const int* ver = ver_idx + (size_t)row * ver_rows + r;
  bf16* pool = pool_v + (size_t)row * pool_rows * HD + lane * 4;
  // ---- the updates from the row's birth on, 32 at a time: which touched the row (one lane per update), then in order
  for (int u0 = u_b; u0 < n_plan; u0 += 32) {
    const int u = u0 + lane;
    bool touched = false;
    int slot = -1;
    if (u < n_plan) {
      touched = u > 0 && ((bits[(size_t)u * words] >> (r & 31)) & 1u);
      if (versions && (touched || u == u_b)) {
        const int vr = plan[u].version_row;
        if (vr >= 0) slot = ver[vr];
      }
    }
    unsigned todo = __ballot_sync(0xffffffffu, touched || u == u_b);
    const unsigned tmask = __ballot_sync(0xffffffffu, touched);
    // the deltas of up to eight touched updates are fetched together
    while (todo) {
      constexpr int NB = 8;
      int src[NB], sl[NB];
      uint2 dl[NB];
      int n = 0;
#pragma unroll
      for (int i = 0; i < NB; ++i) {
        src[i] = todo ? __ffs(todo) - 1 : -1;
        if (todo) { todo &= todo - 1; ++n; }
        sl[i] = src[i] >= 0 ? __shfl_sync(0xffffffffu, slot, src[i]) : -1;
        dl[i] = make_uint2(0u, 0u);
        if (src[i] >= 0 && ((tmask >> src[i]) & 1u) && sl[i] >= 0) dl[i] = *reinterpret_cast<const uint2*>(pool + (size_t)sl[i] * HD);
      }
#pragma unroll
      for (int i = 0; i < NB; ++i) {
        if (i < n) {
          if ((tmask >> src[i]) & 1u) {
            const float2 d0 = unpack_bf16(dl[i].x), d1 = unpack_bf16(dl[i].y);
            x[0] = bf16_round(x[0] + d0.x); x[1] = bf16_round(x[1] + d0.y);
            x[2] = bf16_round(x[2] + d1.x); x[3] = bf16_round(x[3] + d1.y);
          }
          if (sl[i] >= 0) {
            uint2 o;
            view(o);
            *reinterpret_cast<uint2*>(pool + (size_t)sl[i] * HD) = o;
          }
        }
      }
    }
  }
  // ---- the carried state and its final view
  const size_t off = ((size_t)row * mem.capacity + r) * HD + lane * 4;
  uint2 s;
  s.x = pack_bf16(x[0], x[1]);
  s.y = pack_bf16(x[2], x[3]);
  *reinterpret_cast<uint2*>(mem.v_sum + off) = s;
  if (lane == 0) mem.vlen[(size_t)row * mem.capacity + r] = vl;
  uint2 o;
  view(o);
  *reinterpret_cast<uint2*>(mem.v_attn + off) = o;
}

}  // namespace vside

// The value side of one batch after the routing kernel: deltas on the tensor cores, then the per-row walk.
// born: [rows][s_max] token that created each memory row; tbits: [rows][n_plan][ceil(s_max / 32)] scratch.
cudaError_t launch_vside(const LayerDev& L, int batch, long long T, Tensor4 v, Tensor4 gate, const kvm_update_plan* plan_dev,
                         int n_plan, int s_max, MemoryDev mem, bf16* pool_v, long long pool_rows, const int* ver_idx,
                         long long ver_rows, const int* route, const int* born, unsigned* tbits, int* status,
                         uint32_t wait_limit, cudaStream_t stream) {
  using namespace vside;
  const int rows = batch * L.Hkv, C = L.C;
  const int words = ceil_div(s_max, 32);
  {
    Maps maps;
    maps.head_inner = v.sh < v.st ? 1 : 0;
    bool okm;
    if (maps.head_inner) {
      const cuuint64_t dims[4] = {(cuuint64_t)HD, (cuuint64_t)L.Hkv, (cuuint64_t)T, (cuuint64_t)batch};
      const cuuint64_t strides[3] = {(cuuint64_t)v.sh * 2, (cuuint64_t)v.st * 2, (cuuint64_t)v.sb * 2};
      const cuuint32_t box[4] = {64, 1, (cuuint32_t)C, 1};
      okm = encode_bf16_map(&maps.v, v.ptr, 4, dims, strides, box);
    } else {
      const cuuint64_t dims[4] = {(cuuint64_t)HD, (cuuint64_t)T, (cuuint64_t)L.Hkv, (cuuint64_t)batch};
      const cuuint64_t strides[3] = {(cuuint64_t)v.st * 2, (cuuint64_t)v.sh * 2, (cuuint64_t)v.sb * 2};
      const cuuint32_t box[4] = {64, (cuuint32_t)C, 1, 1};
      okm = encode_bf16_map(&maps.v, v.ptr, 4, dims, strides, box);
    }
    if (!okm) return cudaErrorInvalidValue;
    const Layout lay(C, s_max);
    cudaError_t e = cudaFuncSetAttribute(kvm_vdelta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)lay.total);
    if (e != cudaSuccess) return e;
    int dev = 0, n_sm = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    const int n_jobs = rows * (n_plan - 1);
    const int grid = std::max(1, std::min(n_jobs, n_sm));
    kvm_vdelta_kernel<<<grid, kThreads, lay.total, stream>>>(L, gate, plan_dev, n_plan, rows, route, pool_v, pool_rows, ver_idx,
                                                             ver_rows, tbits, words, s_max, status, wait_limit, maps);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  dim3 agrid((unsigned)ceil_div(s_max, kApWarps), rows);
  kvm_vapply_kernel<<<agrid, kApWarps * 32, 0, stream>>>(L, v, gate, plan_dev, n_plan, born, mem, pool_v, pool_rows, ver_idx, ver_rows,
                                                         tbits, words, s_max, status);
  return cudaGetLastError();
}

}  // namespace kvm
