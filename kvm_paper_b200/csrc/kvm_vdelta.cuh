// The value-delta jobs of the memory chain (one job = one (kv row, update)): shared by the stand-alone kernel that runs
// behind the routing kernel and by the spare CTAs of the routing kernel's own launch, which take jobs while the routing
// of later updates is still under way.  Jobs are handed out through a counter in global memory in the order
// (update, kv row); a job may be taken once the routing kernel has published that update for that kv row.
#pragma once

#include "kvm_common.cuh"
#include "kvm_tc.cuh"
#include "kvm_tma_host.cuh"

namespace kvm {
namespace vside {

constexpr int HD = 128;
constexpr int kThreads = 512;         // threads that work on a job (a CTA may have more: the rest stays out)
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
  int job;       // the job thread 0 took for everybody (-1: none)
  int red[16];
};

struct Maps {
  CUtensorMap v;     // the values [B, H, T, D] (dimensions ordered by stride), boxes of 64 elements x C tokens
  int head_inner;
};

// What a job needs.  `progress` (null: every job is ready): per (kv row, CTA of its cluster) the last update whose routes
// and version table the routing kernel has published; `chain_done` / `chain_ctas`: how many routing CTAs have finished and
// how many there are (a CTA of the routing launch stops taking jobs once the routing is over, so that the launch ends
// and the stand-alone kernel behind it takes the rest with every SM).
struct DeltaArgs {
  LayerDev L;
  Tensor4 gate;
  const kvm_update_plan* plan;
  int n_plan, rows;
  const int* route;
  bf16* pool_v;
  long long pool_rows;
  const int* ver_idx;
  long long ver_rows;
  unsigned* tbits;
  int words, s_max;
  int* status;
  uint32_t wait_limit;
  int* queue;            // the next job to hand out
  const int* progress;
  int nc;
  const int* chain_done;
  int chain_ctas;
  // Jobs that a CTA of the routing's launch took but gave back (their update was not published within a short while:
  // such a CTA never holds anything up), taken first by the kernel behind it: the list, its length, the next to take.
  int* given_back;
  int* n_given_back;
  int* given_back_taken;
};

__device__ __forceinline__ bool wait(uint64_t* bar, uint32_t parity, uint32_t limit) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (tc::mbar_try_wait(bar, parity)) return true;
    if (i >= 4096) __nanosleep(100);
  }
  return false;
}
__device__ __forceinline__ int ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// barrier / vote of the kThreads threads that work on jobs (named barrier 1: the CTA may have more threads)
__device__ __forceinline__ void jsync() { asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory"); }
__device__ __forceinline__ bool jvote(bool ok) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %1, 0;\n\t"
      "barrier.cta.red.and.pred q, 1, %2, p;\n\t"
      "selp.b32 %0, 1, 0, q;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)ok), "n"(kThreads)
      : "memory");
  return r != 0;
}

// One thread: take the next job (-1: none left, or the routing is over and this CTA belongs to its launch).
// Jobs are numbered update-major: job j = kv row j % rows of update 1 + j / rows.
__device__ __forceinline__ int take_job(const DeltaArgs& a, int n_jobs) {
  if (a.progress) {
    if (ld_acquire(a.chain_done) >= a.chain_ctas) return -1;  // the routing is over: this launch should end
  } else if (a.given_back) {
    const int i = atomicAdd(a.given_back_taken, 1);
    if (i < *a.n_given_back) return a.given_back[i];
  }
  const int j = atomicAdd(a.queue, 1);
  return j < n_jobs ? j : -1;
}
// One thread: wait until the routing kernel has published job j's update for its kv row.  Jobs are handed out in the
// order in which they become ready, so the wait is short unless this CTA is ahead of the routing; it gives up after
// about a millisecond, or when the routing has ended without publishing the update (false: the job is to be given back).
__device__ __forceinline__ bool job_ready(const DeltaArgs& a, int j) {
  if (a.progress == nullptr) return true;
  const int row = j % a.rows, u = 1 + j / a.rows;
  for (uint32_t spin = 0; spin < 4096u; ++spin) {
    bool ready = true;
    for (int c = 0; c < a.nc && ready; ++c) ready = ld_acquire(a.progress + (size_t)row * a.nc + c) >= u;
    if (ready) return true;
    if (ld_acquire(a.chain_done) >= a.chain_ctas) {  // over: published now, or never (the routing gave up)
      ready = true;
      for (int c = 0; c < a.nc && ready; ++c) ready = ld_acquire(a.progress + (size_t)row * a.nc + c) >= u;
      return ready;
    }
    __nanosleep(300);
  }
  return false;
}

// The job loop of one CTA (its first kThreads threads; `tid` < kThreads).  Returns false if a bounded wait expired.
__device__ __forceinline__ bool delta_jobs(const DeltaArgs& a, const Maps& maps, unsigned char* smem, int tid) {
  const LayerDev& L = a.L;
  const int n_plan = a.n_plan, rows = a.rows, words = a.words, s_max = a.s_max;
  const int C = L.C;
  const Layout lay(C, s_max);
  Bars* bars = reinterpret_cast<Bars*>(smem + lay.bars);
  const int warp = tid >> 5, lane = tid & 31;
  float* gs = reinterpret_cast<float*>(smem + lay.gs);
  unsigned short* stamps = reinterpret_cast<unsigned short*>(smem + lay.rows);
  short* gci = reinterpret_cast<short*>(smem + lay.rows) + ((s_max + 63) & ~31);
  unsigned short* tl = reinterpret_cast<unsigned short*>(smem + lay.tl);
  const int n_jobs = rows * (n_plan - 1);
  if (tid == 0) {
    tc::mbar_init(&bars->full_v, 1);
    tc::mbar_init(&bars->mma_done, 1);
    bars->abort = 0;
    bars->job = take_job(a, n_jobs);
    tc::fence_barrier_init();
  }
  for (int i = tid; i < s_max; i += kThreads) stamps[i] = 0;
  if (warp == 0) tc::tmem_alloc(&bars->tmem_base, kTmemCols);
  tc::tc_fence_before_sync();
  jsync();
  tc::tc_fence_after_sync();
  const uint32_t tmem = bars->tmem_base;
  uint32_t n_v = 0, n_mma = 0;  // uses of the two barriers so far
  unsigned n_mine = 0;          // jobs of this CTA so far (their number stamps the touched rows)
  bool ok = true;

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
  auto has_merges = [&](int j) { return a.plan[1 + j / rows].n_append < C; };
  // the routing decision and the gate of this thread's token of a job
  // (the decisions come from another SM in the same launch when the routing is still under way: read past this SM's L1)
  auto fetch = [&](int j, int& dec, float& g) {
    dec = -1;
    g = 0.f;
    if (j >= 0 && tid < C) {
      const int row = j % rows, u = 1 + j / rows;
      dec = __ldcg(a.route + ((size_t)row * n_plan + u) * C + tid);
      g = __bfloat162float(*a.gate.row(row / L.Hkv, row % L.Hkv, (long long)u * C + tid));
    }
  };
  // the decisions of a job are requested one job ahead when they are all there (the kernel behind the routing); a CTA
  // of the routing's launch asks for them when the job's update has been published
  const bool ahead = a.progress == nullptr;
  int job = bars->job;
  if (tid == 0 && job >= 0 && has_merges(job)) load_values(job);
  int my_next = -1;
  float g_next = 0.f;
  if (ahead) fetch(job, my_next, g_next);
  jsync();  // everybody has read the first job
  while (job >= 0 && ok) {
    const int row = job % rows, u = 1 + job / rows;
    if (!ahead) {
      bool rdy = true;
      if (tid == 0) rdy = job_ready(a, job);
      if (!jvote(rdy)) {
        // give the job back (the kernel behind this launch takes it) and leave; its values may be on their way
        if (has_merges(job)) ok = wait(&bars->full_v, n_v & 1, a.wait_limit);
        if (tid == 0) a.given_back[atomicAdd(a.n_given_back, 1)] = job;
        break;
      }
      fetch(job, my_next, g_next);
    }
    const kvm_update_plan pl = a.plan[u];
    const int S1 = pl.state_before + pl.n_append;
    const bool merges = pl.n_append < C;
    const unsigned short stamp = (unsigned short)(1u + (n_mine++ & 0x7fffu));  // differs from the last 32767 jobs' (rows start at 0)
    // ---- routing decisions and gates of the block; touched rows and their compact order
    const int my = my_next;
    if (tid < C) {
      gs[tid] = g_next;
      if (my >= 0) stamps[my] = stamp;
    }
    jsync();
    int n_touched = 0;
    for (int r0 = 0; r0 < words * 32; r0 += kThreads) {
      const int r = r0 + tid;
      const bool t = r < S1 && stamps[r] == stamp;
      const unsigned bal = __ballot_sync(0xffffffffu, t);
      if (lane == 0) {
        bars->red[warp] = __popc(bal);
        if ((r >> 5) < words) a.tbits[((size_t)row * n_plan + u) * words + (r >> 5)] = bal;
      }
      jsync();
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
      jsync();
    }
    int next = -1;
    if (merges) {
      // ---- one-hot operands: touched row with compact index c in tile c / 128, accumulator lane c % 128
      const int n_tiles = ceil_div(n_touched, 128);  // 1 or 2 (at most C - 1 rows are touched)
      {
        uint4* o = reinterpret_cast<uint4*>(smem + lay.O);
        for (int i = tid; i < n_tiles * C * 16; i += kThreads) o[i] = make_uint4(0, 0, 0, 0);
      }
      // ---- gv = bf16(v * gate) in place (the swizzle permutes 16-byte pieces inside a row: piece i belongs to token (i % 8C) / 8)
      ok = wait(&bars->full_v, n_v & 1, a.wait_limit);
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
      jsync();
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
        slot[t] = t * 128 + ci < n_touched ? __ldcg(a.ver_idx + (size_t)row * a.ver_rows + pl.version_row + tl[t * 128 + ci]) : -1;
      tc::fence_proxy_async();  // the gated values and the one-hot rows -> visible to the tensor core
      tc::tc_fence_before_sync();
      jsync();
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
        // the next job (taken behind the MMAs: the counter is a round trip to L2)
        bars->job = take_job(a, n_jobs);
      }
      ok = ok && wait(&bars->mma_done, n_mma & 1, a.wait_limit);
      ++n_mma;
      jsync();
      next = bars->job;  // -1: none
      if (tid == 0 && next >= 0 && has_merges(next)) load_values(next);  // the values are consumed: the next job's block may land
      if (ahead) fetch(next, my_next, g_next);
      tc::tc_fence_after_sync();
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (t < n_tiles) {
          uint32_t d[32];
          tc::tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(t * 128 + colq * 32), d);
          tc::tmem_ld_wait();
          if (slot[t] >= 0) {
            bf16* dst = a.pool_v + ((size_t)row * a.pool_rows + slot[t]) * HD + colq * 32;
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
    } else {  // nothing was merged (whole block appended): only the bit table
      if (tid == 0) bars->job = take_job(a, n_jobs);
      jsync();
      next = bars->job;
      if (tid == 0 && next >= 0 && has_merges(next)) load_values(next);
      if (ahead) fetch(next, my_next, g_next);
    }
    ok = jvote(ok);  // the accumulators, the one-hot buffers and the job slot are free again
    job = next;
  }
  if (!ok && tid == 0) atomicExch(a.status, KVM_ERR_DEVICE_TIMEOUT);
  if (!ok) {
    for (int k2 = 0; k2 < 64; ++k2) __nanosleep(1000);  // a copy of this CTA may still be in flight
  }
  tc::tc_fence_before_sync();
  jsync();
  if (warp == 0) tc::tmem_dealloc(tmem, kTmemCols);
  return ok;
}

}  // namespace vside
}  // namespace kvm
