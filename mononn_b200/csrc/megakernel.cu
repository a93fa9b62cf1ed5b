// One persistent, table-driven kernel for the whole inference graph (sm_100a).
//
// Replaces the per-graph generated kernel of the reference
// (mononn_engine/codegen/graph_codegen.cc:734-803): instead of emitting CUDA
// text per HLO module, the host fills a stage table (stage_table.h) and this
// kernel interprets it in a single cooperative launch.
//
// Warp roles inside each 256-thread CTA (one CTA per SM):
//   warp 0  weight producer : streams packed weight tiles HBM -> smem ring via TMA.
//                             It never waits for the grid barrier (weights do not
//                             depend on activations), so HBM stays busy across stages.
//   warp 1  activation producer : after the previous stage's grid barrier, TMA-loads
//                             128x64 activation tiles (L2 resident) into the A ring.
//   warp 2  MMA issuer      : tcgen05.mma (kind::f16, fp32 accumulate in TMEM).
//   warps 4-7 epilogue/SIMT : tcgen05.ld -> bias/activation/residual -> global;
//                             softmax of the attention stage; LayerNorm / embedding rows;
//                             grid-barrier arrive.
//
// Grid barrier (replaces mononn_engine/core/gpu/synchronization.cc:45-97): one
// monotonically increasing counter; each CTA adds 1 with release semantics after
// its stores of a stage and polls with acquire until (stage+1)*gridDim arrivals.
// Every wait in this file is bounded; on expiry the kernel records where it gave
// up in KernelStatus and all roles drain and return.
#include <cuda.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "stage_table.h"

namespace mononn {

// ----------------------------------------------------------------------------
// PTX wrappers
// ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, int32_t x, int32_t y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(tmap), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() {
  asm volatile("fence.proxy.async;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  __syncwarp();
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_add_f32x4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c),
               "f"(d)
               : "memory");
}

// K-major, 128-byte-swizzled operand tile: rows of 64 f16 (128 B), 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
  return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) |
         (1ull << 46) | (2ull << 61);
}
// f16 x f16 -> f32, both operands K-major, M = 128.
__device__ __forceinline__ uint32_t umma_idesc_m128(uint32_t n) {
  return (1u << 4) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

// ----------------------------------------------------------------------------
// Shared-memory control block and per-thread context
// ----------------------------------------------------------------------------
struct Ctrl {
  uint64_t a_full[kASlots];
  uint64_t a_empty[kASlots];
  uint64_t b_full[kBSlots];
  uint64_t b_empty[kBSlots];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t group_bar;  // the four epilogue warps (128 arrivals per phase)
  uint32_t tmem_base;
  uint32_t abort_flag;
};

struct Ctx {
  const KernelParams* P;
  Ctrl* ctrl;
  uint32_t a_ring;  // shared addresses
  uint32_t b_ring;
  uint8_t* a_ring_ptr;
  uint32_t stage;   // current stage (for status)
  uint32_t group_phase;  // parity of the next group_bar phase (epilogue warps only)
  uint64_t timeout_ns;
};

__device__ __noinline__ void report_failure(const Ctx& c, uint32_t code, uint32_t where) {
  volatile uint32_t* af = &c.ctrl->abort_flag;
  *af = 1;
  KernelStatus* st = c.P->status;
  if (atomicCAS(&st->code, 0u, code) == 0u) {
    st->stage = c.stage;
    st->cta = blockIdx.x;
    st->where = where;
    __threadfence();
  }
}

// Bounded wait on an mbarrier phase. Returns false when the kernel is aborting.
__device__ __forceinline__ bool mbar_wait(const Ctx& c, uint64_t* bar, uint32_t parity,
                                          uint32_t where) {
  const uint32_t b = smem_u32(bar);
  if (mbar_try_wait(b, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t it = 0;
  for (;;) {
    if (mbar_try_wait(b, parity)) return true;
    if ((++it & 63u) == 0u) {
      if (*reinterpret_cast<volatile uint32_t*>(&c.ctrl->abort_flag)) return false;
      if (globaltimer_ns() - t0 > c.timeout_ns) {
        report_failure(c, ST_MBARRIER_TIMEOUT, where);
        return false;
      }
    }
  }
}

// Bounded wait until every CTA has arrived for all stages before `stage`.
__device__ __forceinline__ bool grid_wait(const Ctx& c, uint32_t stage, uint32_t where) {
  const KernelParams& P = *c.P;
  if (stage == P.stage_begin) return true;
  const uint32_t target = P.epoch_base + (stage - P.stage_begin) * gridDim.x;
  if (static_cast<int32_t>(ld_acquire_gpu(P.barrier) - target) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t it = 0;
  for (;;) {
    if (static_cast<int32_t>(ld_acquire_gpu(P.barrier) - target) >= 0) return true;
    if ((++it & 31u) == 0u) {
      if (*reinterpret_cast<volatile uint32_t*>(&c.ctrl->abort_flag)) return false;
      if (*reinterpret_cast<volatile uint32_t*>(&P.status->code) != 0u) {
        *reinterpret_cast<volatile uint32_t*>(&c.ctrl->abort_flag) = 1;
        return false;
      }
      if (globaltimer_ns() - t0 > c.timeout_ns) {
        report_failure(c, ST_GRID_BARRIER_TIMEOUT, where);
        return false;
      }
    }
  }
}

// Warp-collective variants for the epilogue warps: every lane gets the same answer, so a
// warp never splits around the warp-wide tcgen05.ld that follows.
__device__ __forceinline__ bool mbar_wait_warp(const Ctx& c, uint64_t* bar, uint32_t parity,
                                               uint32_t where) {
  const bool ok = mbar_wait(c, bar, parity, where);
  return __all_sync(0xffffffffu, ok);
}
__device__ __forceinline__ bool grid_wait_warp(const Ctx& c, uint32_t stage, uint32_t where) {
  bool ok = true;
  if ((threadIdx.x & 31u) == 0u) ok = grid_wait(c, stage, where);
  return __all_sync(0xffffffffu, ok);
}
// Barrier across the 128 epilogue threads built on an mbarrier so that, unlike bar.sync,
// the wait is bounded when a warp has already left on the abort path.
__device__ __forceinline__ bool group_sync(Ctx& c, uint32_t where) {
  mbar_arrive(smem_u32(&c.ctrl->group_bar));
  const bool ok = mbar_wait(c, &c.ctrl->group_bar, c.group_phase, where);
  c.group_phase ^= 1u;
  return __all_sync(0xffffffffu, ok);
}

#define WAIT_OR_RETURN(expr) \
  do {                       \
    if (!(expr)) return;     \
  } while (0)

struct Item {
  const OpDesc* op;
  uint32_t local;  // item index inside the op
};

__device__ __forceinline__ Item locate(const KernelParams& P, const StageDesc& st, uint32_t item) {
  const OpDesc* op = P.ops + st.op_begin;
  uint32_t i = item;
  for (uint32_t k = 0; k + 1 < st.op_count && i >= op->n_items; ++k) {
    i -= op->n_items;
    ++op;
  }
  return Item{op, i};
}

struct GemmTile {
  uint32_t mt, nt, ks;
};
__device__ __forceinline__ GemmTile gemm_tile(const OpDesc& op, uint32_t local) {
  GemmTile t;
  t.ks = local % op.k_split;
  const uint32_t r = local / op.k_split;
  t.nt = r % op.n_tiles;
  t.mt = r / op.n_tiles;
  return t;
}

struct AttnTile {
  uint32_t b, h, mt;
};
__device__ __forceinline__ AttnTile attn_tile(const OpDesc& op, uint32_t local) {
  AttnTile t;
  const uint32_t mts = (op.seq + 127u) / 128u;
  t.mt = local % mts;
  const uint32_t r = local / mts;
  t.h = r % op.heads;
  t.b = r / op.heads;
  return t;
}

constexpr uint32_t kAttnASlots = 5;  // Q, K, V^T, P(2)

// ----------------------------------------------------------------------------
// Role: weight producer (warp 0, one lane)
// ----------------------------------------------------------------------------
__device__ void role_weight_producer(Ctx c) {
  const KernelParams& P = *c.P;
  const uint8_t* tmaps = static_cast<const uint8_t*>(P.tmaps);
  uint32_t b_cnt = 0;
  for (uint32_t s = P.stage_begin; s < P.stage_end; ++s) {
    c.stage = s;
    const StageDesc st = P.stages[s];
    for (uint32_t item = blockIdx.x; item < st.n_items; item += gridDim.x) {
      const Item it = locate(P, st, item);
      const OpDesc& op = *it.op;
      if (op.kind != OP_GEMM) continue;
      const GemmTile t = gemm_tile(op, it.local);
      const uint32_t nkb = op.kb_per_split, kbps = op.kb_per_bslot;
      const uint32_t kb_total = op.k_split * nkb;
      const uint32_t row0 = (t.nt * kb_total + t.ks * nkb) * op.n_tile;
      const uint32_t bytes = op.n_tile * kbps * 128u;
      const void* tm = tmaps + static_cast<size_t>(op.tmap_b) * 128u;
      for (uint32_t kb = 0; kb < nkb; kb += kbps) {
        const uint32_t slot = b_cnt % kBSlots, use = b_cnt / kBSlots;
        WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->b_empty[slot], (use & 1u) ^ 1u, 0x100));
        const uint32_t full = smem_u32(&c.ctrl->b_full[slot]);
        mbar_arrive_expect_tx(full, bytes);
        tma_load_2d(c.b_ring + slot * kSlotBytes, tm, 0, static_cast<int32_t>(row0 + kb * op.n_tile),
                    full);
        ++b_cnt;
      }
    }
  }
}

// ----------------------------------------------------------------------------
// Role: activation producer (warp 1, one lane)
// ----------------------------------------------------------------------------
__device__ void role_act_producer(Ctx c) {
  const KernelParams& P = *c.P;
  const uint8_t* tmaps = static_cast<const uint8_t*>(P.tmaps);
  uint32_t a_cnt = 0;
  for (uint32_t s = P.stage_begin; s < P.stage_end; ++s) {
    c.stage = s;
    const StageDesc st = P.stages[s];
    bool waited = false;
    for (uint32_t item = blockIdx.x; item < st.n_items; item += gridDim.x) {
      const Item it = locate(P, st, item);
      const OpDesc& op = *it.op;
      if (op.kind != OP_GEMM && op.kind != OP_ATTENTION) continue;
      if (!waited) {
        WAIT_OR_RETURN(grid_wait(c, s, 0x200));
        fence_proxy_async_all();
        waited = true;
      }
      if (op.kind == OP_GEMM) {
        const GemmTile t = gemm_tile(op, it.local);
        const void* tm = tmaps + static_cast<size_t>(op.tmap_a) * 128u;
        const uint32_t nkb = op.kb_per_split;
        for (uint32_t kb = 0; kb < nkb; ++kb) {
          const uint32_t slot = a_cnt % kASlots, use = a_cnt / kASlots;
          WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->a_empty[slot], (use & 1u) ^ 1u, 0x201));
          const uint32_t full = smem_u32(&c.ctrl->a_full[slot]);
          mbar_arrive_expect_tx(full, kSlotBytes);
          tma_load_2d(c.a_ring + slot * kSlotBytes, tm,
                      static_cast<int32_t>((t.ks * nkb + kb) * 64u),
                      static_cast<int32_t>(t.mt * 128u), full);
          ++a_cnt;
        }
      } else {
        const AttnTile t = attn_tile(op, it.local);
        const void* tm = tmaps + static_cast<size_t>(op.tmap_a) * 128u;
        const void* tmk = tmaps + static_cast<size_t>(op.tmap_b) * 128u;
        const void* tmv = tmaps + static_cast<size_t>(op.tmap_vt) * 128u;
        for (uint32_t j = 0; j < 3; ++j) {
          const uint32_t slot = a_cnt % kASlots, use = a_cnt / kASlots;
          WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->a_empty[slot], (use & 1u) ^ 1u, 0x202));
          const uint32_t full = smem_u32(&c.ctrl->a_full[slot]);
          const uint32_t dst = c.a_ring + slot * kSlotBytes;
          mbar_arrive_expect_tx(full, kSlotBytes);
          if (j == 0) {
            tma_load_2d(dst, tm, static_cast<int32_t>(op.q_col + t.h * 64u),
                        static_cast<int32_t>(t.b * op.seq + t.mt * 128u), full);
          } else if (j == 1) {
            tma_load_2d(dst, tmk, static_cast<int32_t>(op.k_col + t.h * 64u),
                        static_cast<int32_t>(t.b * op.seq), full);
          } else {
            const int32_t y = static_cast<int32_t>((t.b * op.heads + t.h) * 64u);
            tma_load_2d(dst, tmv, 0, y, full);
            tma_load_2d(dst + 8192u, tmv, 64, y, full);
          }
          ++a_cnt;
        }
        a_cnt += 2;  // the two P slots are filled by the softmax warps
      }
    }
  }
}

// ----------------------------------------------------------------------------
// Role: MMA issuer (warp 2, one lane)
// ----------------------------------------------------------------------------
__device__ void role_mma(Ctx c, uint32_t tmem_base) {
  const KernelParams& P = *c.P;
  uint32_t a_cnt = 0, b_cnt = 0, acc_cnt = 0;
  for (uint32_t s = P.stage_begin; s < P.stage_end; ++s) {
    c.stage = s;
    const StageDesc st = P.stages[s];
    for (uint32_t item = blockIdx.x; item < st.n_items; item += gridDim.x) {
      const Item it = locate(P, st, item);
      const OpDesc& op = *it.op;
      if (op.kind == OP_GEMM) {
        const uint32_t nkb = op.kb_per_split, kbps = op.kb_per_bslot;
        const uint32_t buf = acc_cnt & 1u;
        WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->acc_empty[buf], ((acc_cnt >> 1) & 1u) ^ 1u, 0x300));
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * kAccCols;
        const uint32_t idesc = umma_idesc_m128(op.n_tile);
        uint32_t b_slot = 0;
        for (uint32_t kb = 0; kb < nkb; ++kb) {
          const uint32_t sub = kb % kbps;
          if (sub == 0) {
            b_slot = b_cnt % kBSlots;
            WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->b_full[b_slot], (b_cnt / kBSlots) & 1u, 0x301));
          }
          const uint32_t a_slot = a_cnt % kASlots;
          WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->a_full[a_slot], (a_cnt / kASlots) & 1u, 0x302));
          tc_fence_after();
          const uint64_t ad = umma_desc_sw128(c.a_ring + a_slot * kSlotBytes);
          const uint64_t bd =
              umma_desc_sw128(c.b_ring + b_slot * kSlotBytes + sub * op.n_tile * 128u);
#pragma unroll
          for (uint32_t k = 0; k < 4; ++k)
            tc_mma_f16(tmem_d, ad + 2u * k, bd + 2u * k, idesc, (kb | k) != 0u);
          tc_commit(smem_u32(&c.ctrl->a_empty[a_slot]));
          ++a_cnt;
          if (sub + 1 == kbps || kb + 1 == nkb) {
            tc_commit(smem_u32(&c.ctrl->b_empty[b_slot]));
            ++b_cnt;
          }
        }
        tc_commit(smem_u32(&c.ctrl->acc_full[buf]));
        ++acc_cnt;
      } else if (op.kind == OP_ATTENTION) {
        uint32_t slot[kAttnASlots], par[kAttnASlots];
        for (uint32_t j = 0; j < kAttnASlots; ++j) {
          slot[j] = (a_cnt + j) % kASlots;
          par[j] = ((a_cnt + j) / kASlots) & 1u;
        }
        a_cnt += kAttnASlots;
        // S = Q K^T  (128 x 128, K = 64)
        uint32_t buf = acc_cnt & 1u;
        WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->acc_empty[buf], ((acc_cnt >> 1) & 1u) ^ 1u, 0x310));
        WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->a_full[slot[0]], par[0], 0x311));
        WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->a_full[slot[1]], par[1], 0x312));
        tc_fence_after();
        {
          const uint64_t ad = umma_desc_sw128(c.a_ring + slot[0] * kSlotBytes);
          const uint64_t bd = umma_desc_sw128(c.a_ring + slot[1] * kSlotBytes);
          const uint32_t idesc = umma_idesc_m128(128);
#pragma unroll
          for (uint32_t k = 0; k < 4; ++k)
            tc_mma_f16(tmem_base + buf * kAccCols, ad + 2u * k, bd + 2u * k, idesc, k != 0u);
        }
        tc_commit(smem_u32(&c.ctrl->acc_full[buf]));
        ++acc_cnt;
        // O = P V  (128 x 64, K = 128)
        buf = acc_cnt & 1u;
        WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->acc_empty[buf], ((acc_cnt >> 1) & 1u) ^ 1u, 0x313));
        WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->a_full[slot[2]], par[2], 0x314));
        WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->a_full[slot[3]], par[3], 0x315));
        WAIT_OR_RETURN(mbar_wait(c, &c.ctrl->a_full[slot[4]], par[4], 0x316));
        tc_fence_after();
        {
          const uint32_t idesc = umma_idesc_m128(64);
#pragma unroll
          for (uint32_t kb = 0; kb < 2; ++kb) {
            const uint64_t ad = umma_desc_sw128(c.a_ring + slot[3 + kb] * kSlotBytes);
            const uint64_t bd = umma_desc_sw128(c.a_ring + slot[2] * kSlotBytes + kb * 8192u);
#pragma unroll
            for (uint32_t k = 0; k < 4; ++k)
              tc_mma_f16(tmem_base + buf * kAccCols, ad + 2u * k, bd + 2u * k, idesc,
                         (kb | k) != 0u);
          }
        }
        for (uint32_t j = 0; j < kAttnASlots; ++j) tc_commit(smem_u32(&c.ctrl->a_empty[slot[j]]));
        tc_commit(smem_u32(&c.ctrl->acc_full[buf]));
        ++acc_cnt;
      }
    }
  }
}

// ----------------------------------------------------------------------------
// Epilogue / SIMT math
// ----------------------------------------------------------------------------
__device__ __forceinline__ float apply_act(float x, uint32_t act) {
  switch (act) {
    case ACT_GELU_ERF:
      return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
    case ACT_RELU:
      return fmaxf(x, 0.0f);
    case ACT_QUICK_GELU:
      return x / (1.0f + __expf(-1.702f * x));
    case ACT_GELU_TANH: {
      const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.0f + tanhf(u));
    }
    default:
      return x;
  }
}

__device__ __forceinline__ void load_f16x16(const __half* p, float (&o)[16]) {
  const uint4 u0 = __ldg(reinterpret_cast<const uint4*>(p));
  const uint4 u1 = __ldg(reinterpret_cast<const uint4*>(p) + 1);
  const uint32_t w[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    o[2 * i] = f.x;
    o[2 * i + 1] = f.y;
  }
}
// Activations written earlier in this launch: plain (coherent) loads, never the read-only path.
__device__ __forceinline__ void load_f16x16_coherent(const __half* p, float (&o)[16]) {
  const uint4 u0 = __ldcg(reinterpret_cast<const uint4*>(p));
  const uint4 u1 = __ldcg(reinterpret_cast<const uint4*>(p) + 1);
  const uint32_t w[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    o[2 * i] = f.x;
    o[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

__device__ void gemm_epilogue(const Ctx& c, const OpDesc& op, uint32_t local, uint32_t tmem_acc,
                              uint32_t quarter, uint32_t lane) {
  const GemmTile t = gemm_tile(op, local);
  const uint32_t row = quarter * 32u + lane;
  const uint32_t grow = t.mt * 128u + row;
  const bool row_ok = grow < op.M;
  const bool lead = (t.ks == 0);
  const uint32_t n0 = t.nt * op.n_tile;
  const __half* bias = reinterpret_cast<const __half*>(op.p[1]);
  for (uint32_t c0 = 0; c0 < op.n_tile; c0 += 16) {
    float v[16];
    tc_ld16(tmem_acc + ((quarter * 32u) << 16) + c0, v);
    const uint32_t col = n0 + c0;
    if (!row_ok || col >= op.N) continue;
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] *= op.alpha;
    if ((op.flags & F_BIAS) && lead) {
      float b[16];
      load_f16x16(bias + col, b);
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] += b[i];
    }
    if (op.act != ACT_NONE) {
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = apply_act(v[i], op.act);
    }
    if ((op.flags & F_RESID) && lead) {
      if (op.flags & F_RESID_F32) {
        const float4* r = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(op.p[2]) +
                                                          static_cast<size_t>(grow) * op.ldr + col);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float4 x = __ldcg(r + i);
          v[4 * i] += x.x; v[4 * i + 1] += x.y; v[4 * i + 2] += x.z; v[4 * i + 3] += x.w;
        }
      } else {
        float r[16];
        load_f16x16_coherent(
            reinterpret_cast<const __half*>(op.p[2]) + static_cast<size_t>(grow) * op.ldr + col, r);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] += r[i];
      }
    }
    switch (op.out_mode) {
      case OUT_F16: {
        uint4* o = reinterpret_cast<uint4*>(reinterpret_cast<__half*>(op.p[0]) +
                                            static_cast<size_t>(grow) * op.ldo + col);
        o[0] = make_uint4(pack_h2(v[0], v[1]), pack_h2(v[2], v[3]), pack_h2(v[4], v[5]),
                          pack_h2(v[6], v[7]));
        o[1] = make_uint4(pack_h2(v[8], v[9]), pack_h2(v[10], v[11]), pack_h2(v[12], v[13]),
                          pack_h2(v[14], v[15]));
        break;
      }
      case OUT_F16_T: {
        const uint32_t b = grow / op.rows_per_batch, rib = grow % op.rows_per_batch;
        __half* o = reinterpret_cast<__half*>(op.p[0]) +
                    (static_cast<size_t>(b) * op.N + col) * op.ldt + rib;
#pragma unroll
        for (int i = 0; i < 16; ++i) o[static_cast<size_t>(i) * op.ldt] = __float2half_rn(v[i]);
        break;
      }
      case OUT_F32_RED: {
        float* o = reinterpret_cast<float*>(op.p[0]) + static_cast<size_t>(grow) * op.ldo + col;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          red_add_f32x4(o + 4 * i, v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        break;
      }
      default: {
        float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(op.p[0]) +
                                              static_cast<size_t>(grow) * op.ldo + col);
#pragma unroll
        for (int i = 0; i < 4; ++i)
          o[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        break;
      }
    }
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

constexpr int kLnMaxVec = 16;  // float4 chunks per lane -> rows up to 2048 columns

// One warp normalises one row held in registers.
__device__ __forceinline__ void layernorm_row_store(float4 (&x)[kLnMaxVec], uint32_t nvec,
                                                    uint32_t cols, uint32_t lane, float eps,
                                                    const __half* gamma, const __half* beta,
                                                    __half* out) {
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < kLnMaxVec; ++i)
    if (i * 32u + lane < nvec) s += x[i].x + x[i].y + x[i].z + x[i].w;
  const float mean = warp_sum(s) / static_cast<float>(cols);
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < kLnMaxVec; ++i)
    if (i * 32u + lane < nvec) {
      const float a = x[i].x - mean, b = x[i].y - mean, cc = x[i].z - mean, d = x[i].w - mean;
      q += a * a + b * b + cc * cc + d * d;
    }
  const float rstd = rsqrtf(warp_sum(q) / static_cast<float>(cols) + eps);
#pragma unroll
  for (int i = 0; i < kLnMaxVec; ++i) {
    const uint32_t vi = i * 32u + lane;
    if (vi < nvec) {
      const uint2 g = __ldg(reinterpret_cast<const uint2*>(gamma) + vi);
      const uint2 b = __ldg(reinterpret_cast<const uint2*>(beta) + vi);
      const float2 g0 = __half22float2(*reinterpret_cast<const __half2*>(&g.x));
      const float2 g1 = __half22float2(*reinterpret_cast<const __half2*>(&g.y));
      const float2 b0 = __half22float2(*reinterpret_cast<const __half2*>(&b.x));
      const float2 b1 = __half22float2(*reinterpret_cast<const __half2*>(&b.y));
      uint2 o;
      o.x = pack_h2((x[i].x - mean) * rstd * g0.x + b0.x, (x[i].y - mean) * rstd * g0.y + b0.y);
      o.y = pack_h2((x[i].z - mean) * rstd * g1.x + b1.x, (x[i].w - mean) * rstd * g1.y + b1.y);
      reinterpret_cast<uint2*>(out)[vi] = o;
    }
  }
}

__device__ __forceinline__ float4 h4_to_f4(uint2 u) {
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
  return make_float4(a.x, a.y, b.x, b.y);
}

__device__ void layernorm_item(const OpDesc& op, uint32_t local, uint32_t warp_in_group,
                               uint32_t lane) {
  const uint32_t row = local * 4u + warp_in_group;
  if (row >= op.rows) return;
  const uint32_t nvec = op.cols / 4u;
  float4 x[kLnMaxVec];
  if (op.flags & F_SRC_F32) {
    float4* src = reinterpret_cast<float4*>(reinterpret_cast<float*>(op.p[1]) +
                                            static_cast<size_t>(row) * op.lds);
#pragma unroll
    for (int i = 0; i < kLnMaxVec; ++i) {
      const uint32_t vi = i * 32u + lane;
      if (vi < nvec) {
        x[i] = __ldcg(src + vi);
        if (op.flags & F_ZERO_SRC) src[vi] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
  } else {
    const uint2* src = reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(op.p[1]) +
                                                      static_cast<size_t>(row) * op.lds);
#pragma unroll
    for (int i = 0; i < kLnMaxVec; ++i) {
      const uint32_t vi = i * 32u + lane;
      if (vi < nvec) x[i] = h4_to_f4(__ldcg(src + vi));
    }
  }
  if (op.flags & F_RESID) {
    const uint2* r = reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(op.p[4]) +
                                                    static_cast<size_t>(row) * op.ldr);
#pragma unroll
    for (int i = 0; i < kLnMaxVec; ++i) {
      const uint32_t vi = i * 32u + lane;
      if (vi < nvec) {
        const float4 f = h4_to_f4(__ldcg(r + vi));
        x[i].x += f.x; x[i].y += f.y; x[i].z += f.z; x[i].w += f.w;
      }
    }
  }
  layernorm_row_store(x, nvec, op.cols, lane, op.eps, reinterpret_cast<const __half*>(op.p[2]),
                      reinterpret_cast<const __half*>(op.p[3]),
                      reinterpret_cast<__half*>(op.p[0]) + static_cast<size_t>(row) * op.ldo);
}

__device__ void embed_item(const OpDesc& op, uint32_t local, uint32_t warp_in_group,
                           uint32_t lane) {
  const uint32_t row = local * 4u + warp_in_group;
  if (row >= op.rows) return;
  const uint32_t nvec = op.cols / 4u;
  const int32_t id = reinterpret_cast<const int32_t*>(op.p[1])[row];
  const uint32_t pos = row % op.seq;
  const uint2* w = reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(op.p[3]) +
                                                  static_cast<int64_t>(id) * op.cols);
  const uint2* pe = reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(op.p[4]) +
                                                   static_cast<size_t>(pos) * op.cols);
  const uint2* te = nullptr;
  if (op.flags & F_TYPE_IDS) {
    const int32_t ty = reinterpret_cast<const int32_t*>(op.p[2])[row];
    te = reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(op.p[5]) +
                                        static_cast<int64_t>(ty) * op.cols);
  }
  float4 x[kLnMaxVec];
#pragma unroll
  for (int i = 0; i < kLnMaxVec; ++i) {
    const uint32_t vi = i * 32u + lane;
    if (vi < nvec) {
      float4 a = h4_to_f4(__ldg(w + vi));
      const float4 b = h4_to_f4(__ldg(pe + vi));
      a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
      if (te) {
        const float4 t = h4_to_f4(__ldg(te + vi));
        a.x += t.x; a.y += t.y; a.z += t.z; a.w += t.w;
      }
      x[i] = a;
    }
  }
  layernorm_row_store(x, nvec, op.cols, lane, op.eps, reinterpret_cast<const __half*>(op.p[6]),
                      reinterpret_cast<const __half*>(op.p[7]),
                      reinterpret_cast<__half*>(op.p[0]) + static_cast<size_t>(row) * op.ldo);
  if ((op.flags & F_MASK_BIAS) && lane == 0) {
    const int32_t m = reinterpret_cast<const int32_t*>(op.q[0])[row];
    reinterpret_cast<float*>(op.q[1])[row] = (1.0f - static_cast<float>(m)) * -10000.0f;
  }
}

// Softmax + output of one attention tile; thread `row` owns query row `row`.
__device__ bool attention_simt(Ctx& c, const OpDesc& op, uint32_t local, uint32_t tmem_base,
                               uint32_t& a_cnt, uint32_t& acc_cnt, uint32_t quarter, uint32_t lane,
                               uint32_t tid_in_group) {
  const AttnTile t = attn_tile(op, local);
  const uint32_t row = quarter * 32u + lane;
  const uint32_t qrow = t.mt * 128u + row;  // query index inside the sequence
  const uint32_t slotP0 = (a_cnt + 3) % kASlots, slotP1 = (a_cnt + 4) % kASlots;
  const uint32_t parP0 = ((a_cnt + 3) / kASlots) & 1u, parP1 = ((a_cnt + 4) / kASlots) & 1u;
  a_cnt += kAttnASlots;

  uint32_t buf = acc_cnt & 1u;
  if (!mbar_wait_warp(c, &c.ctrl->acc_full[buf], (acc_cnt >> 1) & 1u, 0x410)) return false;
  tc_fence_after();
  const uint32_t tS = tmem_base + buf * kAccCols + ((quarter * 32u) << 16);
  const float* mb = (op.flags & F_MASK_BIAS)
                        ? reinterpret_cast<const float*>(op.p[1]) + static_cast<size_t>(t.b) * op.seq
                        : nullptr;
  const uint32_t n_keys = op.seq < 128u ? op.seq : 128u;
  const bool causal = (op.flags & F_CAUSAL) != 0u;
  // pass 1: row maximum of scale*s + bias over the valid keys
  float mx = -3.0e38f;
  for (uint32_t c0 = 0; c0 < 128u; c0 += 16) {
    float v[16];
    tc_ld16(tS + c0, v);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t key = c0 + i;
      if (key < n_keys && !(causal && key > qrow)) {
        const float z = v[i] * op.alpha + (mb ? __ldcg(mb + key) : 0.f);
        mx = fmaxf(mx, z);
      }
    }
  }
  // the P slots must be free before they are overwritten
  if (!mbar_wait_warp(c, &c.ctrl->a_empty[slotP0], parP0 ^ 1u, 0x411)) return false;
  if (!mbar_wait_warp(c, &c.ctrl->a_empty[slotP1], parP1 ^ 1u, 0x412)) return false;
  // pass 2: p = exp(z - max), row sum, P tile in the swizzled K-major operand layout
  float sum = 0.f;
  for (uint32_t c0 = 0; c0 < 128u; c0 += 16) {
    float v[16];
    tc_ld16(tS + c0, v);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t key = c0 + i;
      float p = 0.f;
      if (key < n_keys && !(causal && key > qrow)) {
        const float z = v[i] * op.alpha + (mb ? __ldcg(mb + key) : 0.f);
        p = __expf(z - mx);
      }
      // sum what the tensor core will actually multiply (the f16-rounded value)
      v[i] = __half2float(__float2half_rn(p));
      sum += v[i];
    }
    uint8_t* tile = c.a_ring_ptr + ((c0 < 64u) ? slotP0 : slotP1) * kSlotBytes;
    const uint32_t chunk = (c0 & 63u) >> 3;  // 16-byte chunk index inside the 128-byte row
    uint4* d0 = reinterpret_cast<uint4*>(tile + row * 128u + (((chunk) ^ (row & 7u)) << 4));
    uint4* d1 = reinterpret_cast<uint4*>(tile + row * 128u + (((chunk + 1u) ^ (row & 7u)) << 4));
    *d0 = make_uint4(pack_h2(v[0], v[1]), pack_h2(v[2], v[3]), pack_h2(v[4], v[5]),
                     pack_h2(v[6], v[7]));
    *d1 = make_uint4(pack_h2(v[8], v[9]), pack_h2(v[10], v[11]), pack_h2(v[12], v[13]),
                     pack_h2(v[14], v[15]));
  }
  fence_proxy_async_smem();
  tc_fence_before();
  if (!group_sync(c, 0x414)) return false;
  if (tid_in_group == 0) {
    mbar_arrive(smem_u32(&c.ctrl->a_full[slotP0]));
    mbar_arrive(smem_u32(&c.ctrl->a_full[slotP1]));
  }
  mbar_arrive(smem_u32(&c.ctrl->acc_empty[buf]));
  ++acc_cnt;

  // O = P V
  buf = acc_cnt & 1u;
  if (!mbar_wait_warp(c, &c.ctrl->acc_full[buf], (acc_cnt >> 1) & 1u, 0x413)) return false;
  tc_fence_after();
  const uint32_t tO = tmem_base + buf * kAccCols + ((quarter * 32u) << 16);
  const float inv = 1.0f / sum;
  const bool row_ok = qrow < op.seq;
  __half* out = reinterpret_cast<__half*>(op.p[0]) +
                (static_cast<size_t>(t.b) * op.seq + qrow) * op.ldo + t.h * 64u;
  for (uint32_t c0 = 0; c0 < 64u; c0 += 16) {
    float v[16];
    tc_ld16(tO + c0, v);
    if (row_ok) {
      uint4* o = reinterpret_cast<uint4*>(out + c0);
      o[0] = make_uint4(pack_h2(v[0] * inv, v[1] * inv), pack_h2(v[2] * inv, v[3] * inv),
                        pack_h2(v[4] * inv, v[5] * inv), pack_h2(v[6] * inv, v[7] * inv));
      o[1] = make_uint4(pack_h2(v[8] * inv, v[9] * inv), pack_h2(v[10] * inv, v[11] * inv),
                        pack_h2(v[12] * inv, v[13] * inv), pack_h2(v[14] * inv, v[15] * inv));
    }
  }
  tc_fence_before();
  mbar_arrive(smem_u32(&c.ctrl->acc_empty[buf]));
  ++acc_cnt;
  return true;
}

// ----------------------------------------------------------------------------
// Role: epilogue + SIMT stages + grid barrier (warps 4..7)
// ----------------------------------------------------------------------------
__device__ void role_simt(Ctx c, uint32_t tmem_base, uint32_t tid_in_group) {
  const KernelParams& P = *c.P;
  const uint32_t quarter = tid_in_group >> 5, lane = tid_in_group & 31u;
  uint32_t a_cnt = 0, acc_cnt = 0;
  for (uint32_t s = P.stage_begin; s < P.stage_end; ++s) {
    c.stage = s;
    const StageDesc st = P.stages[s];
    // All CTAs must have finished the previous stage before this CTA reads its
    // results or arrives for this stage.
    WAIT_OR_RETURN(grid_wait_warp(c, s, 0x400));
    if (P.stamps != nullptr && blockIdx.x == 0 && tid_in_group == 0)
      P.stamps[s - P.stage_begin] = globaltimer_ns();
    for (uint32_t item = blockIdx.x; item < st.n_items; item += gridDim.x) {
      const Item it = locate(P, st, item);
      const OpDesc& op = *it.op;
      switch (op.kind) {
        case OP_GEMM: {
          const uint32_t buf = acc_cnt & 1u;
          WAIT_OR_RETURN(mbar_wait_warp(c, &c.ctrl->acc_full[buf], (acc_cnt >> 1) & 1u, 0x401));
          tc_fence_after();
          gemm_epilogue(c, op, it.local, tmem_base + buf * kAccCols, quarter, lane);
          tc_fence_before();
          mbar_arrive(smem_u32(&c.ctrl->acc_empty[buf]));
          ++acc_cnt;
          a_cnt += op.kb_per_split;
          break;
        }
        case OP_ATTENTION:
          WAIT_OR_RETURN(
              attention_simt(c, op, it.local, tmem_base, a_cnt, acc_cnt, quarter, lane, tid_in_group));
          break;
        case OP_LAYERNORM:
          layernorm_item(op, it.local, quarter, lane);
          break;
        case OP_EMBED:
          embed_item(op, it.local, quarter, lane);
          break;
        default:
          break;
      }
    }
    // publish this CTA's stores of the stage, then arrive
    fence_proxy_async_all();
    WAIT_OR_RETURN(group_sync(c, 0x402));
    if (tid_in_group == 0) {
      __threadfence();
      red_release_gpu_add(P.barrier, 1u);
    }
  }
  if (P.stamps != nullptr && blockIdx.x == 0 && tid_in_group == 0)
    P.stamps[P.stage_end - P.stage_begin] = globaltimer_ns();
}

// ----------------------------------------------------------------------------
// Kernel
// ----------------------------------------------------------------------------
extern "C" __global__ void __launch_bounds__(kThreads, 1)
mononn_megakernel(const __grid_constant__ KernelParams P) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw & 1023u)) & 1023u;
  uint8_t* base = smem_raw + pad;
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(base + (kASlots + kBSlots) * kSlotBytes);

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  if (threadIdx.x == 0) {
    for (uint32_t i = 0; i < kASlots; ++i) {
      mbar_init(smem_u32(&ctrl->a_full[i]), 1);
      mbar_init(smem_u32(&ctrl->a_empty[i]), 1);
    }
    for (uint32_t i = 0; i < kBSlots; ++i) {
      mbar_init(smem_u32(&ctrl->b_full[i]), 1);
      mbar_init(smem_u32(&ctrl->b_empty[i]), 1);
    }
    for (uint32_t i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&ctrl->acc_full[i]), 1);
      mbar_init(smem_u32(&ctrl->acc_empty[i]), 128);
    }
    mbar_init(smem_u32(&ctrl->group_bar), 128);
    ctrl->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&ctrl->tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&ctrl->tmem_base);

  Ctx c;
  c.P = &P;
  c.ctrl = ctrl;
  c.a_ring = smem_u32(base);
  c.b_ring = c.a_ring + kASlots * kSlotBytes;
  c.a_ring_ptr = base;
  c.stage = P.stage_begin;
  c.group_phase = 0;
  c.timeout_ns = static_cast<uint64_t>(P.timeout_us) * 1000ull;

  if (warp == 0) {
    if (lane == 0) role_weight_producer(c);
  } else if (warp == 1) {
    if (lane == 0) role_act_producer(c);
  } else if (warp == 2) {
    if (lane == 0) role_mma(c, tmem_base);
  } else if (warp >= 4) {
    role_simt(c, tmem_base, threadIdx.x - 128u);
  }
  __syncwarp();

  // Teardown. On the abort path give copies and MMAs still in flight time to land
  // before the shared memory and TMEM they target are released.
  if (*reinterpret_cast<volatile uint32_t*>(&ctrl->abort_flag)) __nanosleep(2000000);
  tc_fence_before();
  __syncthreads();
  if (*reinterpret_cast<volatile uint32_t*>(&ctrl->abort_flag)) __nanosleep(2000000);
  if (warp == 2) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTmemCols)
                 : "memory");
  }
}

}  // namespace mononn
