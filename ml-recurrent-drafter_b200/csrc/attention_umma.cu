// Tree-masked flash attention on the 5th-generation tensor cores (head_dim 128, bf16).
//
// One CTA serves 128 queries of one (batch row, head): normally every packed tree token of the row.
//   warps 0, 6  TMA producers (one elected lane each): warp 0 loads the K tiles of 64 keys, warp 6 the V
//               tiles (two 64-column boxes each, 128-byte swizzle, no multicast), each into its own
//               two-stage ring; the Q tile and the first two K and V tiles are requested by thread 0 as
//               soon as the barriers exist, before the TMEM allocation.  A K stage is free as soon as QK^T of
//               its tile is done, a V stage after PV; the producers wait on the same completion
//               barriers the softmax uses (one commit per product);
//   warp 1      MMA issuer (one elected thread):
//                 S = Q K^T   tcgen05.mma, A = Q and B = K from shared memory (both K-major),
//                             accumulator S[128 x 64] in TMEM;
//                 O_t = P V   tcgen05.mma, A = P (bf16) read from TMEM, B = V from shared memory as
//                             an MN-major operand (V rows are keys, head_dim contiguous);
//   warps 2-5   softmax: thread r owns query row r (= TMEM lane r): tcgen05.ld of its S row, one
//               64-bit visibility word per tile (cached prefix, causal or prefix-tree bitmask), a
//               running max that only moves when exceeded by more than 2^6, p = 2^(s*c - m*c) by one
//               FFMA + ex2.approx, P written back to TMEM with tcgen05.st.  O accumulates in TMEM
//               across tiles; a warp rescales its O rows (tcgen05.ld / st) only on the tiles where
//               one of its rows' running max moved.
// QK of tile t+1 overlaps the softmax and PV of tile t; P is double-buffered in TMEM so that the
// softmax of tile t does not wait for PV of tile t-1 before writing P; two CTAs fit on an SM (105 KB
// of shared memory, 256 TMEM columns each) and overlap each other's latencies.  With n_split > 1
// a CTA walks only its share of the key tiles and leaves an unnormalised partial for the merge
// kernel at the end of this file.
//
// Every mbarrier wait is bounded; on give-up the kernel records a code in *status, stops issuing,
// lets outstanding bulk copies land, frees its TMEM and returns.
#include <cuda.h>

#include "rd_common.cuh"

namespace {

constexpr int HD = 128;
constexpr int BMQ = 128;  // queries per CTA
constexpr int BNK = 64;   // keys per tile
constexpr int kThreads = 224;
constexpr int kSubTile = 64 * 128;            // bytes of a [64 rows x 64 bf16] box = 8 KB
constexpr int kQBytes = BMQ * HD * 2;         // 32 KB: two [128 x 64] boxes
constexpr int kKVStage = 2 * BNK * HD * 2;    // 32 KB: K (2 boxes) then V (2 boxes)
constexpr int kStages = 2;
constexpr int kMaxMaskWords = 16;
constexpr int kMaskBytes = BMQ * kMaxMaskWords * 4;  // the tile's bitmask rows
constexpr int kSmemBytes = kQBytes + kStages * kKVStage + kMaskBytes + 1024 + 256;
// TMEM columns
constexpr float kMaxSlack = 6.0f;  // log2 units the tile max may exceed the running max without moving it
constexpr uint32_t kColS = 0;     // S: 64 fp32 columns
constexpr uint32_t kColP = 64;    // P: two buffers of 64 bf16 = 32 columns each
constexpr uint32_t kColO = 128;   // O: 128 fp32 columns, accumulated over the tiles
constexpr uint32_t kTmemCols = 256;

struct AttnPlan {
  CUtensorMap map_q;  // [m_max, nh*128] box 64 x 128
  CUtensorMap map_k;  // [B*nkv*max_len, 128] box 64 x 64
  CUtensorMap map_v;
  int nh, nkv, max_len, B, m_max;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// One attempt: the hardware may suspend the thread until the phase completes or a time limit of its own
// expires, so a waiter costs no issue slots while it waits and wakes as soon as the barrier flips.
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait (one second).  Returns false when it gave up or when another role already aborted.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_test(bar, parity)) return true;
  const uint64_t t0 = global_ns();
  for (;;) {
    if (mbar_try(bar, parity)) return true;
    if (*abort_flag) return false;
    if (global_ns() - t0 > 1000000000ull) return false;
  }
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
// K-major tile, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}
// MN-major tile, 128-byte swizzle: 64 contiguous MN elements per 128-byte row, consecutive K rows
// 128 bytes apart, 8-row groups `sbo` bytes apart, the next 64 MN elements `lbo` bytes away.
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) | ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// fp32 accumulator, bf16 operands, M = 128
__device__ __forceinline__ uint32_t idesc_f16(int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void umma_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d),
      "l"(a), "l"(b), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void umma_ts(uint32_t d, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d),
      "r"(a_tmem), "l"(b), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
      "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
      "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
      "r"(r[31])
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(kThreads, 2)
    attention_umma_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                          const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                          const int32_t* __restrict__ row_start, const int32_t* __restrict__ kv_begin,
                          const int32_t* __restrict__ base_len, int nh, int nkv, int max_len, int mode,
                          const uint32_t* __restrict__ tree_mask, int mask_words, float scale_log2, int32_t* status,
                          int n_split, float* __restrict__ partial) {
  const int b = blockIdx.z, h = blockIdx.y;
  rd::pdl_launch_dependents();
  if (threadIdx.x == 0) {
    // the descriptors are kernel parameters: their fetch may start before the dependency wait
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
  }
  rd::pdl_wait();  // row_start, Q and the new K/V rows come from the kernels before this one
  const int rs = row_start[b];
  const int n_new = row_start[b + 1] - rs;
  const int q0 = ((int)blockIdx.x / n_split) * BMQ;
  const int split = (int)blockIdx.x % n_split;  // this CTA's share of the key tiles (1 share = the whole row)
  if (q0 >= n_new) return;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sKV = smem + kQBytes;
  uint32_t* sMask = reinterpret_cast<uint32_t*>(smem + kQBytes + kStages * kKVStage);  // [128][mask_words]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kQBytes + kStages * kKVStage + kMaskBytes);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* v_full = bars + 3;    // [2]
  uint64_t* s_full = bars + 5;    // [2]: QK^T of even / odd tiles done; also frees that tile's K stage
  uint64_t* s_empty = bars + 7;
  uint64_t* p_full = bars + 8;
  uint64_t* o_full = bars + 9;    // [2]: PV of even / odd tiles done; also frees that tile's V stage
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int base = base_len[b];
  const int hk = h / (nh / nkv);
  const int kv_end = (mode == RD_ATTN_CAUSAL) ? base + min(n_new, q0 + BMQ) : base + n_new;
  const int all_tiles = (kv_end + BNK - 1) / BNK;
  const int per_split = (all_tiles + n_split - 1) / n_split;
  const int t_begin = split * per_split;  // first key tile of this CTA
  const int n_tiles = max(0, min(per_split, all_tiles - t_begin));
  if (n_split > 1 && n_tiles == 0) {
    // nothing to do for this share: leave an empty partial (max = -inf, sum = 0) for the merge
    const int r = (int)threadIdx.x, qi = q0 + r;
    if (r < BMQ && qi < n_new) {
      float* ml = partial + (((int64_t)(rs + qi) * nh + h) * n_split + split) * (HD + 2) + HD;
      ml[0] = -INFINITY;
      ml[1] = 0.f;
    }
    return;
  }
  const int kv_row0 = (b * nkv + hk) * max_len + kv_begin[b];  // row of key 0 in the [B*nkv*max_len, 128] view

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&o_full[s], 1);
    }
    mbar_init(s_empty, 4);
    mbar_init(p_full, 4);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // The first loads (Q and the first ring's worth of K and V tiles) go out here, before the TMEM
    // allocation and the block-wide barrier below: a short chain of key tiles spends a large part of its
    // life waiting for this first data.
    mbar_expect_tx(q_full, kQBytes);
    tma_load_2d(sQ, &map_q, q_full, h * HD, rs + q0);
    tma_load_2d(sQ + BMQ * 128, &map_q, q_full, h * HD + 64, rs + q0);
    for (int t = 0; t < kStages && t < n_tiles; ++t) {
      const int row = kv_row0 + (t_begin + t) * BNK;
      uint8_t* dk = sKV + t * kKVStage;
      mbar_expect_tx(&k_full[t], 2 * kSubTile);
      tma_load_2d(dk, &map_k, &k_full[t], 0, row);
      tma_load_2d(dk + kSubTile, &map_k, &k_full[t], 64, row);
    }
    for (int t = 0; t < kStages && t < n_tiles; ++t) {
      const int row = kv_row0 + (t_begin + t) * BNK;
      uint8_t* dv = sKV + t * kKVStage + 2 * kSubTile;
      mbar_expect_tx(&v_full[t], 2 * kSubTile);
      tma_load_2d(dv, &map_v, &v_full[t], 0, row);
      tma_load_2d(dv + kSubTile, &map_v, &v_full[t], 64, row);
    }
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 || warp == 6) {
    // ---------------- TMA producers: warp 0 = Q and the K ring, warp 6 = the V ring ----------------
    if (lane == 0) {
      const bool is_k = warp == 0;
      uint64_t* full = is_k ? k_full : v_full;
      // a stage is free when the product that read it is done: QK^T of tile t-2 for K, PV of tile t-2
      // for V.  Each of these barriers completes once per two tiles, so a parity wait is unambiguous.
      uint64_t* done = is_k ? s_full : o_full;
      const CUtensorMap* map = is_k ? &map_k : &map_v;
      bool ok = true;
      for (int t = kStages; ok && t < n_tiles; ++t) {  // tiles 0 .. kStages-1 were requested at set-up
        const int s = t & 1;
        if (!mbar_wait(&done[s], ((t - 2) >> 1) & 1, abort_flag)) {
          ok = false;
          break;
        }
        uint8_t* dst = sKV + s * kKVStage + (is_k ? 0 : 2 * kSubTile);
        mbar_expect_tx(&full[s], 2 * kSubTile);
        const int row = kv_row0 + (t_begin + t) * BNK;
        tma_load_2d(dst, map, &full[s], 0, row);
        tma_load_2d(dst + kSubTile, map, &full[s], 64, row);
      }
      if (!ok) {
        if (atomicCAS((int*)abort_flag, 0, 1) == 0 && status) atomicExch(status, 21);
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc_qk = idesc_f16(BNK, false);
      const uint32_t idesc_pv = idesc_f16(HD, true);
      const uint32_t tS = tmem_base + kColS, tP = tmem_base + kColP, tO = tmem_base + kColO;
      bool ok = mbar_wait(q_full, 0, abort_flag);
      auto issue_qk = [&](int t) {
        const uint8_t* sK = sKV + (t & 1) * kKVStage;
#pragma unroll
        for (int kd = 0; kd < HD / 16; ++kd) {
          const uint64_t da = desc_k_major(smem_u32(sQ + (kd >> 2) * (BMQ * 128) + (kd & 3) * 32));
          const uint64_t db = desc_k_major(smem_u32(sK + (kd >> 2) * kSubTile + (kd & 3) * 32));
          umma_ss(tS, da, db, idesc_qk, kd != 0);
        }
        umma_commit(&s_full[t & 1]);  // S is ready; the K stage is free once this product is done
      };
      if (ok && n_tiles > 0) {
        ok = mbar_wait(&k_full[0], 0, abort_flag);
        if (ok) {
          tc_fence_after();
          issue_qk(0);
        }
      }
      for (int t = 0; ok && t < n_tiles; ++t) {
        if (t + 1 < n_tiles) {
          // S of tile t has been read by the softmax threads -> QK of tile t+1 may overwrite it
          if (!mbar_wait(&k_full[(t + 1) & 1], ((t + 1) >> 1) & 1, abort_flag)) {
            ok = false;
            break;
          }
          if (!mbar_wait(s_empty, t & 1, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          issue_qk(t + 1);
        }
        // P of tile t is in TMEM (and O has been rescaled where needed); V of tile t has landed
        if (!mbar_wait(p_full, t & 1, abort_flag)) {
          ok = false;
          break;
        }
        if (!mbar_wait(&v_full[t & 1], (t >> 1) & 1, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint8_t* sV = sKV + (t & 1) * kKVStage + 2 * kSubTile;
#pragma unroll
        for (int ks = 0; ks < BNK / 16; ++ks) {
          // V: keys are the K dimension (rows of 128 bytes), head_dim the MN dimension: two 64-wide
          // halves kSubTile bytes apart, 8-key groups 1024 bytes apart; 16 keys per MMA = 2048 bytes
          const uint64_t dv = desc_mn_major(smem_u32(sV + ks * 2048), kSubTile, 1024);
          umma_ts(tO, tP + (t & 1) * 32 + ks * 8, dv, idesc_pv, (t | ks) != 0);
        }
        umma_commit(&o_full[t & 1]);  // O holds tile t; its P buffer and V stage are free
      }
      if (!ok && atomicCAS((int*)abort_flag, 0, 1) == 0 && status) atomicExch(status, 22);
    }
  } else {
    // ---------------- softmax: thread <-> query row ----------------
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;  // row of the tile = TMEM lane
    const int qi = q0 + r;              // query index within the batch row
    const bool live = qi < n_new;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    if (mode == RD_ATTN_TREE) {
      for (int w = 0; w < mask_words; ++w) sMask[r * mask_words + w] = live ? tree_mask[(int64_t)(rs + qi) * mask_words + w] : 0u;
    }
    const uint32_t* my_mask = sMask + r * mask_words;  // written and read by this thread only
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    int site = 0;  // which wait gave up (reported in the status word)
    for (int t = 0; ok && t < n_tiles; ++t) {
      if (!mbar_wait(&s_full[t & 1], (t >> 1) & 1, abort_flag)) {
        ok = false;
        site = 1;
        break;
      }
      tc_fence_after();
      uint32_t sb[64];
      tmem_ld32(lane_addr + kColS, sb);
      tmem_ld32(lane_addr + kColS + 32, sb + 32);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_empty);
      // visibility of the tile's 64 keys for this row as one 64-bit word
      const int j0 = (t_begin + t) * BNK;
      uint64_t vis;
      if (j0 + BNK <= base) {
        vis = ~0ull;  // the whole tile lies in the cached prefix
      } else {
        const int off = j0 - base;  // index of the tile's first key among the new tokens (may be negative)
        uint64_t nb;                // visibility of new tokens [max(off,0), ...) aligned to bit max(-off,0)
        const int first = off > 0 ? off : 0;
        if (mode == RD_ATTN_CAUSAL) {
          // new token jn is visible iff jn <= qi
          const int n_vis = qi - first + 1;
          nb = n_vis >= 64 ? ~0ull : (n_vis <= 0 ? 0ull : ((1ull << n_vis) - 1ull));
        } else {
          const int w = first >> 5, sh = first & 31;
          const uint64_t lo = w < mask_words ? my_mask[w] : 0u;
          const uint64_t mid = w + 1 < mask_words ? my_mask[w + 1] : 0u;
          const uint64_t hi = w + 2 < mask_words ? my_mask[w + 2] : 0u;
          nb = ((lo | (mid << 32)) >> sh) | (sh ? (hi << (64 - sh)) : 0ull);
        }
        vis = off >= 0 ? nb : ((nb << (-off)) | ((1ull << (-off)) - 1ull));
      }
      if (j0 + BNK > kv_end) {
        const int n_in = kv_end - j0;  // 1..63 keys of the tile exist
        vis &= (n_in <= 0) ? 0ull : ((1ull << n_in) - 1ull);
      }
      // Running max over the RAW scores (the scale is positive), masked keys set to -inf first.
      // exp2 then takes one FFMA per element: p = 2^(s*scale - m*scale).
      float mx = -INFINITY;
      if (__all_sync(0xffffffffu, vis == ~0ull)) {
#pragma unroll
        for (int i = 0; i < 64; i += 2) mx = fmaxf(mx, fmaxf(__uint_as_float(sb[i]), __uint_as_float(sb[i + 1])));
      } else {
        const uint32_t vlo = (uint32_t)vis, vhi = (uint32_t)(vis >> 32);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (!((vlo >> i) & 1u)) sb[i] = 0xff800000u;
          if (!((vhi >> i) & 1u)) sb[32 + i] = 0xff800000u;
        }
#pragma unroll
        for (int i = 0; i < 64; i += 2) mx = fmaxf(mx, fmaxf(__uint_as_float(sb[i]), __uint_as_float(sb[i + 1])));
      }
      // Lazy running max (in log2 units): it only moves when the tile's max exceeds it by more than
      // kMaxSlack, so P stays <= 2^kMaxSlack and O is rescaled rarely; l and O use the same max.
      const float mx2 = mx * scale_log2;
      const bool moved = mx2 > m_run + kMaxSlack;  // also true for the first visible key (m_run = -inf)
      const float m_new = moved ? mx2 : m_run;
      const float alpha = (m_run == -INFINITY) ? 0.f : ex2_approx(m_run - m_new);
      const bool rescale = moved && (m_run != -INFINITY);
      m_run = m_new;
      const float neg_m = (m_new == -INFINITY) ? 0.f : -m_new;
      float rowsum0 = 0.f, rowsum1 = 0.f;
      uint32_t pb[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float p0 = ex2_approx(fmaf(__uint_as_float(sb[2 * i]), scale_log2, neg_m));
        const float p1 = ex2_approx(fmaf(__uint_as_float(sb[2 * i + 1]), scale_log2, neg_m));
        rowsum0 += p0;
        rowsum1 += p1;
        pb[i] = pack_bf16(p0, p1);
      }
      l_run = l_run * (moved ? alpha : 1.0f) + (rowsum0 + rowsum1);
      // P buffer t&1 was last read by PV of tile t-2, seen complete before this warp's arrival for tile t-1
      if (__any_sync(0xffffffffu, rescale)) {
        // O must be quiescent while it is rescaled: PV of tile t-1 has to be complete
        if (!mbar_wait(&o_full[(t - 1) & 1], ((t - 1) >> 1) & 1, abort_flag)) {
          ok = false;
          site = 3;
          break;
        }
        tc_fence_after();
        const float a = rescale ? alpha : 1.0f;
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t ob[32];
          tmem_ld32(lane_addr + kColO + c * 32, ob);
#pragma unroll
          for (int i = 0; i < 32; ++i) ob[i] = __float_as_uint(__uint_as_float(ob[i]) * a);
          tmem_st32(lane_addr + kColO + c * 32, ob);
        }
      }
      tmem_st32(lane_addr + kColP + (t & 1) * 32, pb);
      tc_fence_before();
      // The arrival for tile t must not be possible before the MMA thread has consumed the barrier's
      // phase for tile t-1: the thread issues QK of tile t before it looks at that phase, so without
      // this wait a fast softmax could complete two phases between two of its polls, and a parity
      // wait cannot tell phase t-1 from phase t+1.  PV of tile t-1 complete implies it was consumed
      // (and that no warp's arrival for tile t can be counted into the phase of tile t-1).
      if (t >= 1 && !mbar_wait(&o_full[(t - 1) & 1], ((t - 1) >> 1) & 1, abort_flag)) {
        ok = false;
        site = 4;
        break;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok && n_tiles > 0) {
      ok = mbar_wait(&o_full[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1, abort_flag);
      if (!ok) site = 5;
    }
    if (ok && n_split > 1) {
      // partial result of this share: unnormalised O (relative to m_run), then m_run and l_run
      tc_fence_after();
      float* dstp = partial + (((int64_t)(rs + qi) * nh + h) * n_split + split) * (HD + 2);
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t ob[32];
        tmem_ld32(lane_addr + kColO + c * 32, ob);
        if (live) {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            *reinterpret_cast<float2*>(dstp + c * 32 + 2 * i) = make_float2(__uint_as_float(ob[2 * i]), __uint_as_float(ob[2 * i + 1]));
        }
      }
      if (live) {
        dstp[HD] = m_run;
        dstp[HD + 1] = l_run;
      }
    } else if (ok) {
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
      uint4* dst = reinterpret_cast<uint4*>(out + ((int64_t)(rs + qi) * nh + h) * HD);
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t ob[32];
        tmem_ld32(lane_addr + kColO + c * 32, ob);
        if (live) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 pk;
            pk.x = pack_bf16(__uint_as_float(ob[8 * i]) * inv, __uint_as_float(ob[8 * i + 1]) * inv);
            pk.y = pack_bf16(__uint_as_float(ob[8 * i + 2]) * inv, __uint_as_float(ob[8 * i + 3]) * inv);
            pk.z = pack_bf16(__uint_as_float(ob[8 * i + 4]) * inv, __uint_as_float(ob[8 * i + 5]) * inv);
            pk.w = pack_bf16(__uint_as_float(ob[8 * i + 6]) * inv, __uint_as_float(ob[8 * i + 7]) * inv);
            dst[c * 4 + i] = pk;
          }
        }
      }
    }
    if (!ok && lane == 0 && atomicCAS((int*)abort_flag, 0, 1) == 0 && status) atomicExch(status, 2300 + site);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// Merge of the shares of a split launch: out = sum_s O_s 2^(m_s - m) / sum_s l_s 2^(m_s - m).
__global__ void __launch_bounds__(HD) attention_merge_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out,
                                                             const int32_t* __restrict__ row_start, int B, int nh, int n_split) {
  const int tok = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  if (tok >= row_start[B]) return;
  const float* p = partial + ((int64_t)tok * nh + h) * n_split * (HD + 2);
  float m = -INFINITY;
  for (int s = 0; s < n_split; ++s) m = fmaxf(m, p[s * (HD + 2) + HD]);
  float acc = 0.f, l = 0.f;
  for (int s = 0; s < n_split; ++s) {
    const float ms = p[s * (HD + 2) + HD];
    const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - m);
    acc += w * p[s * (HD + 2) + d];
    l += w * p[s * (HD + 2) + HD + 1];
  }
  out[((int64_t)tok * nh + h) * HD + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}
bool make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld_elems, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld_elems * 2};
  cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

extern "C" void* rd_attention_plan_create(const void* q, int m_max, const void* k_cache, const void* v_cache, int B, int nh,
                                          int nkv, int hd, int max_len) {
  if (!q || !k_cache || !v_cache || m_max < 1 || B < 1 || nh < 1 || nkv < 1 || nh % nkv || hd != HD || max_len < 1) return nullptr;
  if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) return nullptr;
  AttnPlan* p = new AttnPlan();
  p->nh = nh;
  p->nkv = nkv;
  p->max_len = max_len;
  p->B = B;
  p->m_max = m_max;
  const int64_t kv_rows = (int64_t)B * nkv * max_len;
  if (!make_map(&p->map_q, q, m_max, (int64_t)nh * HD, (int64_t)nh * HD, BMQ) ||
      !make_map(&p->map_k, k_cache, kv_rows, HD, HD, BNK) || !make_map(&p->map_v, v_cache, kv_rows, HD, HD, BNK)) {
    delete p;
    return nullptr;
  }
  return p;
}

extern "C" void rd_attention_plan_destroy(void* plan) { delete static_cast<AttnPlan*>(plan); }

extern "C" int64_t rd_attention_split_workspace_bytes(int m_max, int nh, int n_split);

static int attention_tc_launch(const void* plan, void* out, const int32_t* row_start, const int32_t* kv_begin,
                               const int32_t* base_len, int max_new, int mode, const uint32_t* tree_mask, int mask_words,
                               int n_split, void* workspace, int64_t workspace_bytes, int32_t* status, void* stream) {
  RD_REQUIRE(plan && out && row_start && kv_begin && base_len, RD_ERR_ARG);
  RD_REQUIRE(mode == RD_ATTN_CAUSAL || (mode == RD_ATTN_TREE && tree_mask && mask_words >= 1 && mask_words <= kMaxMaskWords),
             RD_ERR_ARG);
  RD_REQUIRE(max_new >= 1 && n_split >= 1 && n_split <= RD_ATTN_MAX_SPLIT, RD_ERR_SIZE);
  RD_REQUIRE(((uintptr_t)out & 15) == 0, RD_ERR_ALIGN);
  const AttnPlan* p = static_cast<const AttnPlan*>(plan);
  RD_REQUIRE(p->B <= 65535 && p->nh <= 65535, RD_ERR_SIZE);
  if (n_split > 1) {
    RD_REQUIRE(workspace && ((uintptr_t)workspace & 15) == 0, RD_ERR_ARG);
    RD_REQUIRE(workspace_bytes >= rd_attention_split_workspace_bytes(p->m_max, p->nh, n_split), RD_ERR_CAPACITY);
  }
  auto kern = attention_umma_kernel;
  static bool smem_set = false;  // set once, so that steady-state launches are pure launches
  if (!smem_set) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    smem_set = true;
  }
  dim3 grid(((max_new + BMQ - 1) / BMQ) * n_split, p->nh, p->B);
  const float scale_log2 = 1.4426950408889634f / sqrtf((float)HD);
  cudaError_t err = rd::launch_chained(kern, grid, dim3(kThreads), kSmemBytes, (cudaStream_t)stream, 1, p->map_q, p->map_k, p->map_v,
                                       (__nv_bfloat16*)out, row_start, kv_begin, base_len, p->nh, p->nkv, p->max_len, mode,
                                       tree_mask, mask_words, scale_log2, status, n_split, (float*)workspace);
  RD_CHECK_CHAINED(err);
  if (n_split > 1) {
    attention_merge_kernel<<<dim3(p->m_max, p->nh), HD, 0, (cudaStream_t)stream>>>((const float*)workspace, (__nv_bfloat16*)out,
                                                                                 row_start, p->B, p->nh, n_split);
  }
  RD_CHECK_LAUNCH();
  return RD_OK;
}

extern "C" int64_t rd_attention_split_workspace_bytes(int m_max, int nh, int n_split) {
  return (int64_t)m_max * nh * n_split * (HD + 2) * (int64_t)sizeof(float);
}

extern "C" int rd_attention_tc(const void* plan, void* out, const int32_t* row_start, const int32_t* kv_begin,
                               const int32_t* base_len, int max_new, int mode, const uint32_t* tree_mask, int mask_words,
                               int32_t* status, void* stream) {
  return attention_tc_launch(plan, out, row_start, kv_begin, base_len, max_new, mode, tree_mask, mask_words, 1, nullptr, 0,
                             status, stream);
}

extern "C" int rd_attention_tc_split(const void* plan, void* out, const int32_t* row_start, const int32_t* kv_begin,
                                     const int32_t* base_len, int max_new, int mode, const uint32_t* tree_mask, int mask_words,
                                     int n_split, void* workspace, int64_t workspace_bytes, int32_t* status, void* stream) {
  return attention_tc_launch(plan, out, row_start, kv_begin, base_len, max_new, mode, tree_mask, mask_words, n_split, workspace,
                             workspace_bytes, status, stream);
}
