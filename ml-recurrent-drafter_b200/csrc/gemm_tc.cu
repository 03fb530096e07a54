// C = epilogue(A * W^T), bf16 operands, fp32 accumulation on the 5th-generation tensor cores.
//
// The decode step has few activation rows (M = packed tree tokens, a few hundred to ~1500, known
// only on the device) and large weights, so the WEIGHT rows ride the MMA's M dimension and the
// tokens its N dimension: N may be any multiple of 16 up to 256, chosen per tile at run time, so the
// token rows are split into equal chunks with almost no padding (M = 900 costs 912 columns instead
// of 1024 rows).  The accumulator tile is C^T: TMEM lane = output feature, TMEM column = token.
//
// gemm_tc_pair_kernel is the kernel of the hot path (every projection with at least 256 output
// features): a persistent kernel, one CTA per SM, CTAs paired in clusters of two that share one
// tcgen05.mma.cta_group::2 of 256 weight rows x (up to 256) tokens x 16:
//   warp 0     TMA producer in BOTH CTAs: cp.async.bulk.tensor loads (128-byte swizzle, never
//              multicast) of this CTA's 128 weight rows and of its HALF of the token tile (one box
//              of 32/64/96/128 rows, whichever the chunk's half fills), six stages of 32 KB; both
//              CTAs' loads complete on the leader's mbarrier;
//   warp 1     MMA issuer, leader CTA only: one elected thread issues the MMAs for the pair into
//              one of two TMEM accumulator buffers (each CTA's TMEM receives its 128 rows) and
//              frees a stage / publishes an accumulator with ONE tcgen05.commit whose arrival is
//              delivered to the barrier of both CTAs;
//   warps 2-5  epilogue in both CTAs: tcgen05.ld of the accumulator (each warp its own 32 TMEM
//              lanes), the fused element-wise part (bias / SiLU / SwiGLU / residual / rotary
//              embedding + cache append / arg-max or slice maxima over the vocabulary), a transpose
//              through shared memory after which groups of lanes share token rows, so that every
//              16-byte residual read and store instruction covers whole rows; inputs of the block
//              loop that come from global memory (residual, rotary positions, bias) are staged
//              ahead of it (cp.async or shared memory): a global load in flight makes the waits for
//              the transposition's shared-memory words wait for it as well.  Overlapped with the next
//              tile's main loop through the second accumulator buffer; the peer's epilogue frees the
//              accumulator with remote mbarrier arrives.
// gemm_tc_kernel is the single-CTA form of the same design (cta_group::1, 128 weight rows per tile,
// four stages) for matrices with fewer than 256 output features.
// Tiles are walked weight-tile-major so that the CTAs running at the same time share W tiles
// through L2; GEMMs with few weight tiles cut the tokens finer so that every CTA pair has a tile.
//
// Every mbarrier wait is bounded: when a wait gives up the kernel records a code in *status,
// stops issuing work, lets outstanding bulk copies land, meets its peer at the final cluster
// barrier, frees its TMEM and returns.
#include <cuda.h>
#include <stdlib.h>

#include "rd_common.cuh"

namespace {

constexpr int BM = 128;       // weight rows per tile (MMA M)
constexpr int kMaxChunk = 256;  // tokens per tile (MMA N), multiple of 16
constexpr int kTokBox = 32;     // granularity of the pair kernel's token boxes (rows)
constexpr int BK = 64;        // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;
constexpr uint64_t kWaitLimitNs = 1000000000ull;  // a wait that lasts a second gives up

// Experiment switch: 0 forces the single-CTA kernel (environment RD_GEMM_PAIRS=0, read once).
static int g_use_pairs = [] {
  const char* v = getenv("RD_GEMM_PAIRS");
  return (v && v[0] == '0') ? 0 : 1;
}();

// Experiment builds only (-DRD_GEMM_TIMING; the shipped library carries none of this): acc[0] +=
// nanoseconds CTA 0 spent between its dependency wait and its last tile, acc[1] += 2*M*N*K of the
// launch.  CTA (pair) 0 owns the largest share of the tiles, so its lifetime is the kernel's duration
// without launch latency and without the perturbation of event records between dependent launches.
#ifdef RD_GEMM_TIMING
__device__ unsigned long long* g_gemm_timing = nullptr;
#define RD_TIMING_BEGIN()                                                                                      \
  unsigned long long* const timing = (blockIdx.x == 0 && threadIdx.x == 0) ? g_gemm_timing : nullptr;           \
  const uint64_t t_begin = timing ? global_ns() : 0
#define RD_TIMING_END(M, N, K)                                                                                 \
  if (timing) {                                                                                                \
    atomicAdd(timing, (unsigned long long)(global_ns() - t_begin));                                            \
    atomicAdd(timing + 1, 2ull * (unsigned long long)(M) * (unsigned long long)(N) * (unsigned long long)(K)); \
  }
#else
#define RD_TIMING_BEGIN() do { } while (0)
#define RD_TIMING_END(M, N, K) do { } while (0)
#endif

// Token-operand descriptors of the pair kernel, one per box height (multiples of kTokBox rows up to a CTA's 128).
struct TokMaps {
  CUtensorMap m[4];
};

struct GemmPlan {
  CUtensorMap map_a;    // activations [m_max, K], box 64 x 128 (single-CTA kernel)
  TokMaps maps_a;       // the same tensor in boxes of 64 x 32/64/96/128: the pair kernel fetches only the rows its chunk fills
  CUtensorMap map_w;  // weights [N, K], box 64 x 128
  int m_max, N, K;
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
// One attempt: the hardware may suspend the thread until the phase completes or a time limit of its
// own expires, so a waiter wakes as soon as the barrier flips instead of at its next poll.
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
// Bounded wait (kWaitLimitNs).  Returns false when it gave up or when another role already aborted.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_test(bar, parity)) return true;
  const uint64_t t0 = global_ns();
  for (;;) {
    if (mbar_try(bar, parity)) return true;
    if (*abort_flag) return false;
    if (global_ns() - t0 > kWaitLimitNs) return false;
  }
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}

// K-major operand tile with 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);  // start address, 16-byte units
  d |= (uint64_t)1 << 16;                      // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;            // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                      // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                      // 128-byte swizzle
  return d;
}

__device__ __forceinline__ uint32_t umma_instr_desc(int n) {
  // fp32 accumulator, bf16 A and B, both K-major, M = 128, N = n (multiple of 16, <= 256)
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

// Token chunking shared by all roles: n_chunks equal chunks of `chunk` tokens (a multiple of 16).
// The fewest chunks that respect the 256-token MMA limit are used unless that leaves compute units
// (CTAs or CTA pairs) idle: a GEMM with few weight tiles (N = 4096) then cuts the tokens finer so
// that about one tile exists per unit.  Finer chunks than that cost more than they balance: every
// chunk is one more pass over its weight tile, with a tile's fixed costs (gate/up at 761 tokens: 115 us
// with 3 chunks of 256 in 3.5 rounds of tiles, 135 us with 4 of 192, 150 us with 6 of 128, although both
// leave fewer idle tile slots).
struct Chunking {
  int n_chunks, chunk;
};
__device__ __forceinline__ Chunking make_chunking(int M, int w_units, int avail_units) {
  Chunking c;
  c.n_chunks = (M + kMaxChunk - 1) / kMaxChunk;
  if (c.n_chunks < 1) c.n_chunks = 1;
  if (w_units * c.n_chunks < avail_units) {
    int n = avail_units / w_units;             // tiles <= units: a single, fuller wave
    const int n_cap = (M + 63) / 64;           // keep chunks of at least ~64 tokens
    if (n > n_cap) n = n_cap;
    if (n > c.n_chunks) c.n_chunks = n;
  }
  const int per = (M + c.n_chunks - 1) / c.n_chunks;
  c.chunk = ((per + 15) / 16) * 16;
  if (c.chunk < 16) c.chunk = 16;
  c.n_chunks = (M + c.chunk - 1) / c.chunk;    // rounding up to 16 may have emptied the last chunk
  if (c.n_chunks < 1) c.n_chunks = 1;
  return c;
}
// MMA N of chunk ci: its live tokens rounded up to 16
__device__ __forceinline__ int chunk_cols(const Chunking& c, int ci, int M) {
  int live = M - ci * c.chunk;
  if (live > c.chunk) live = c.chunk;
  if (live < 1) live = 1;
  return ((live + 15) / 16) * 16;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
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

struct EpiArgs {
  void* C;
  int64_t ldc;
  const __nv_bfloat16* bias;
  const void* R;
  int64_t ldr;
  // kEpiQkvRope only: the QKV projection whose epilogue applies the rotary embedding and writes
  // Q rows [tok, head*128 + d] and the K/V cache rows of the token's slot (head_dim 128, bf16)
  __nv_bfloat16* q_out;
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
  const int32_t* tok_row;
  const int32_t* tok_pos;
  const int32_t* tok_slot;
  const float* cos_t;
  const float* sin_t;
  int n_pos, nh, nkv, max_len;
  // LlamaRMSNorm folded into the two GEMMs around it (optional; bf16 output, N a multiple of 32).
  // Producer (residual epilogues, gamma != nullptr): besides C the kernel writes C2 = bf16(C) * gamma and, per token
  // and 128-feature slice (a CTA's rows), the sum of squares of the rounded C values to
  // ss_out[token * ss_out_ld + slice]: no atomics, so the statistics are the same bits from launch to launch.
  // Consumer (SwiGLU and QKV-rope epilogues, ss_in != nullptr): the A rows are such a C2 (scaled by gamma, not
  // normalised); the accumulator row of token t is multiplied by 1 / sqrt(sum_slices ss_in[t][slice] / norm_dim + eps),
  // the slices added in ascending order, before the rest of the epilogue.
  const __nv_bfloat16* gamma;
  __nv_bfloat16* C2;
  int64_t ldc2;
  float* ss_out;
  int64_t ss_out_ld;
  const float* ss_in;
  int64_t ss_in_ld;
  int ss_slices;
  float norm_dim, norm_eps;
  // kEpiArgmax / kEpiSliceMax only: per (32-feature slice, token) partial results, laid out [slice][part_ld]
  float* part_val;               // kEpiSliceMax: largest stored value
  unsigned long long* part_key;  // kEpiArgmax: (order-preserving key of the largest logit) << 32 | ~(first id holding it)
  int64_t part_ld;
};

constexpr int kEpiQkvRope = 6;  // internal epilogue code (not one of RD_EPI_*): reached through rd_gemm_bf16_tc_qkv_rope
// LM head of the greedy verify step: no output matrix; every epilogue warp reduces its 32 output features
// (vocabulary ids) of each token to (largest logit, first id holding it) and a small kernel merges the slices
constexpr int kEpiArgmax = 7;
// plain output plus the largest stored value of every (32-feature slice, token): lets the vocabulary top-k
// that follows find its threshold from the slice maxima and read only the slices that can hold kept entries
constexpr int kEpiSliceMax = 8;

constexpr int kScrLd = 36;  // floats per scratch row: 16-byte aligned rows, conflict-free float4 reads

// Element-wise part of the epilogue in accumulator layout (lane = output feature n, i = token).
template <int EPI>
__device__ __forceinline__ void epilogue_math(float* v, const EpiArgs& e, int n, int N, bool swiglu_here, float bias) {
  if (EPI == RD_EPI_BIAS || EPI == RD_EPI_BIAS_SILU || EPI == RD_EPI_BIAS_SILU_RES) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] += bias;
  }
  if (EPI == RD_EPI_BIAS_SILU || EPI == RD_EPI_BIAS_SILU_RES) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = rd::silu_f(v[i]);
  }
  if (EPI == RD_EPI_SWIGLU && swiglu_here) {
    // feature-per-lane stores only (the vector path forms the product after the transpose):
    // weight rows (2i, 2i+1) = (gate_i, up_i) sit in adjacent lanes; even lanes keep the product
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float up = __shfl_xor_sync(0xffffffffu, v[i], 1);
      v[i] = rd::silu_f(v[i]) * up;
    }
  }
}

// How the lanes of an epilogue warp share the 32 tokens x kOut output features of a block when they read the
// residual and write the result: every access is 16 bytes, the kLanes lanes of a group cover one token's
// kOut features (64 contiguous bytes in bf16, 128 in fp32; half of that after SwiGLU), and the warp's groups
// take kRows tokens per pass.  An instruction then touches kRows lines (4 to 16) instead of the 32 it would
// with one token row per lane, which is what bounded the epilogue: the load/store unit handles one line of a
// warp instruction at a time.
template <bool OUT_F32, int kOut>
struct EpiLanes {
  static constexpr int kPer = OUT_F32 ? 4 : 8;   // output features per 16-byte access
  static constexpr int kLanes = kOut / kPer;     // lanes per token row: 4 (bf16), 8 (fp32), 2 / 4 after SwiGLU
  static constexpr int kRows = 32 / kLanes;      // token rows per pass
  static constexpr int kPasses = kLanes;         // passes per 32-token block
};

// Residual values of a block in that arrangement: q[p] = the 16 bytes this lane adds in pass p.
template <bool OUT_F32, int kOut>
struct ResidualRegs {
  using G = EpiLanes<OUT_F32, kOut>;
  uint4 q[G::kPasses];
  __device__ __forceinline__ void load(const EpiArgs& e, int tok0, int n0, int tok_limit, int lane) {
    const int sub = lane % G::kLanes, row0 = lane / G::kLanes;
    constexpr int esz = OUT_F32 ? 4 : 2;
    const char* base = (const char*)e.R + ((int64_t)(tok0 + row0) * e.ldr + n0 + sub * G::kPer) * esz;
#pragma unroll
    for (int p = 0; p < G::kPasses; ++p)
      if (tok0 + row0 + p * G::kRows < tok_limit)
        q[p] = *reinterpret_cast<const uint4*>(base + (int64_t)p * G::kRows * e.ldr * esz);
  }
  // bf16 residual through shared memory: request() starts asynchronous copies of the block's 16-byte pieces into
  // this warp's staging buffer (every lane copies the pieces it will add itself: slot p * 32 + lane), take() waits for
  // them and moves them to registers.  Unlike register loads the copies are not tracked by the load scoreboards, so
  // the waits for the shared-memory words of the transposition do not wait for them: with the next block's
  // residual in flight as ordinary loads each block paid most of an L2 latency.  `after`: a register the copies are
  // issued after (the last word taken from the buffer they overwrite).
  __device__ __forceinline__ void request(const EpiArgs& e, int tok0, int n0, int tok_limit, int lane, uint4* buf,
                                          uint32_t after) const {
    const int sub = lane % G::kLanes, row0 = lane / G::kLanes;
    const __nv_bfloat16* base = (const __nv_bfloat16*)e.R + (int64_t)(tok0 + row0) * e.ldr + n0 + sub * G::kPer;
#pragma unroll
    for (int p = 0; p < G::kPasses; ++p)
      if (tok0 + row0 + p * G::kRows < tok_limit)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(buf + p * 32 + lane)),
                     "l"(base + (int64_t)p * G::kRows * e.ldr), "r"(after)
                     : "memory");
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  __device__ __forceinline__ void take(const uint4* buf, int lane) {
    asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
    for (int p = 0; p < G::kPasses; ++p) q[p] = buf[p * 32 + lane];
  }
  __device__ __forceinline__ void add_to(int p, float* o) const {
    if (OUT_F32) {
      o[0] += __uint_as_float(q[p].x);
      o[1] += __uint_as_float(q[p].y);
      o[2] += __uint_as_float(q[p].z);
      o[3] += __uint_as_float(q[p].w);
    } else {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q[p]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        o[2 * j] += f.x;
        o[2 * j + 1] += f.y;
      }
    }
  }
};

// One 32-token block of a tile.  v: accumulator values in (lane = feature, i = token) layout after
// epilogue_math.  The block is transposed through this warp's scratch (row = token) and read back in the
// EpiLanes arrangement, so that the residual is read and the result written with 16-byte accesses that
// cover whole token rows.  `vec_ok` is false for ragged feature ranges or unaligned outputs: plain stores then.
template <int EPI, bool OUT_F32>
__device__ __forceinline__ void epilogue_block(float* v, const EpiArgs& e, float* scr, int lane, int n_warp0, int tok0,
                                               int tok_limit, int N, bool vec_ok,
                                               const ResidualRegs<OUT_F32, (EPI == RD_EPI_SWIGLU ? 16 : 32)>& res,
                                               const float* s_scale, uint4 gamma8, float* ss_red_block) {
  constexpr int kOut = (EPI == RD_EPI_SWIGLU) ? 16 : 32;  // output features per token of this warp
  constexpr bool kRes = (EPI == RD_EPI_BIAS_SILU_RES || EPI == RD_EPI_RES);
  using G = EpiLanes<OUT_F32, kOut>;
  const int out0 = (EPI == RD_EPI_SWIGLU) ? (n_warp0 >> 1) : n_warp0;  // first output column of the warp
  if (!vec_ok) {
    // feature-per-lane fallback
    const int n = n_warp0 + lane;
    const bool writer = (EPI == RD_EPI_SWIGLU) ? ((lane & 1) == 0 && n + 1 < N) : (n < N);
    const int col = (EPI == RD_EPI_SWIGLU) ? (n >> 1) : n;
    if (writer) {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int tok = tok0 + i;
        if (tok < tok_limit) {
          float o = v[i];
          if (OUT_F32) {
            if (kRes) o += ((const float*)e.R)[(int64_t)tok * e.ldr + col];
            ((float*)e.C)[(int64_t)tok * e.ldc + col] = o;
          } else {
            if (kRes) o += __bfloat162float(((const __nv_bfloat16*)e.R)[(int64_t)tok * e.ldr + col]);
            ((__nv_bfloat16*)e.C)[(int64_t)tok * e.ldc + col] = __float2bfloat16_rn(o);
          }
        }
      }
    }
    return;
  }
  // transpose: scr[token i][feature]
#pragma unroll
  for (int i = 0; i < 32; ++i) scr[i * kScrLd + lane] = v[i];
  __syncwarp();
  const int sub = lane % G::kLanes, row0 = lane / G::kLanes;
  float* const ss_red = ss_red_block + ((n_warp0 >> 5) & 3) * 32;  // this warp's row of the reduction buffer
  float o[G::kPasses][G::kPer];
  if (EPI == RD_EPI_SWIGLU) {
    // the token's 32 features are 16 (gate, up) pairs: one SiLU per output, no lane exchange.  The SiLUs of the
    // block are evaluated stage by stage (all exponentials, then all quotients) to keep the special-function
    // unit's latency off the critical path.
    float g[G::kPasses][G::kPer], u[G::kPasses][G::kPer];
#pragma unroll
    for (int p = 0; p < G::kPasses; ++p) {
      const float* src = scr + (row0 + p * G::kRows) * kScrLd + sub * 2 * G::kPer;
#pragma unroll
      for (int j = 0; j < G::kPer / 2; ++j) {
        const float4 f = *reinterpret_cast<const float4*>(src + 4 * j);
        g[p][2 * j] = f.x;
        u[p][2 * j] = f.y;
        g[p][2 * j + 1] = f.z;
        u[p][2 * j + 1] = f.w;
      }
    }
    if (s_scale != nullptr) {
      // folded RMS norm: gate and up of a token are scaled by the token's 1 / rms first
#pragma unroll
      for (int p = 0; p < G::kPasses; ++p) {
        const float sc = s_scale[row0 + p * G::kRows];
#pragma unroll
        for (int j = 0; j < G::kPer; ++j) g[p][j] *= sc, u[p][j] *= sc;
      }
    }
#pragma unroll
    for (int p = 0; p < G::kPasses; ++p)
#pragma unroll
      for (int j = 0; j < G::kPer; ++j) o[p][j] = __expf(-g[p][j]);
#pragma unroll
    for (int p = 0; p < G::kPasses; ++p)
#pragma unroll
      for (int j = 0; j < G::kPer; ++j) o[p][j] = __fdividef(g[p][j], 1.0f + o[p][j]) * u[p][j];
  } else {
#pragma unroll
    for (int p = 0; p < G::kPasses; ++p) {
      const float* src = scr + (row0 + p * G::kRows) * kScrLd + sub * G::kPer;
#pragma unroll
      for (int j = 0; j < G::kPer / 4; ++j) {
        const float4 f = *reinterpret_cast<const float4*>(src + 4 * j);
        o[p][4 * j] = f.x;
        o[p][4 * j + 1] = f.y;
        o[p][4 * j + 2] = f.z;
        o[p][4 * j + 3] = f.w;
      }
    }
  }
  __syncwarp();  // the scratch is reused by the next block
  constexpr int esz = OUT_F32 ? 4 : 2;
  char* dst0 = (char*)e.C + ((int64_t)(tok0 + row0) * e.ldc + out0 + sub * G::kPer) * esz;
#pragma unroll
  for (int p = 0; p < G::kPasses; ++p) {
    const int tok = tok0 + row0 + p * G::kRows;
    const bool live = tok < tok_limit;
    float smax = -INFINITY;  // kEpiSliceMax: largest value of the token's 32 features AS STORED
    float ss_part = 0.f;     // folded RMS norm: this lane's share of the token's sum of squares
    if (live) {
      if (kRes) res.add_to(p, o[p]);
      uint4 pk;
      if (OUT_F32) {
        pk = make_uint4(__float_as_uint(o[p][0]), __float_as_uint(o[p][1]), __float_as_uint(o[p][2]), __float_as_uint(o[p][3]));
        if (EPI == kEpiSliceMax) smax = fmaxf(fmaxf(o[p][0], o[p][1]), fmaxf(o[p][2], o[p][3]));
      } else {
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          h[t] = __floats2bfloat162_rn(o[p][2 * t], o[p][2 * t + 1]);
          if (EPI == kEpiSliceMax) {
            const float2 r = __bfloat1622float2(h[t]);
            smax = fmaxf(smax, fmaxf(r.x, r.y));
          }
        }
      }
      *reinterpret_cast<uint4*>(dst0 + (int64_t)p * G::kRows * e.ldc * esz) = pk;
      if (kRes && !OUT_F32 && e.gamma != nullptr) {
        // producer side of the folded RMS norm: statistics and the next GEMM's operand come from the ROUNDED row
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&pk);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gamma8);
        uint4 pk2;
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&pk2);
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float2 f = __bfloat1622float2(h[t]);
          const float2 gm = __bfloat1622float2(g2[t]);
          ss_part += f.x * f.x + f.y * f.y;
          h2[t] = __floats2bfloat162_rn(f.x * gm.x, f.y * gm.y);
        }
        *reinterpret_cast<uint4*>(e.C2 + (int64_t)tok * e.ldc2 + out0 + sub * G::kPer) = pk2;
      }
    }
    if (kRes && !OUT_F32 && e.gamma != nullptr) {
      // the lanes of a group hold the pieces of one token row; the warp's share of the row goes to the reduction buffer
#pragma unroll
      for (int d = 1; d < G::kLanes; d <<= 1) ss_part += __shfl_xor_sync(0xffffffffu, ss_part, d);
      if (sub == 0) ss_red[row0 + p * G::kRows] = live ? ss_part : 0.f;
    }
    if (EPI == kEpiSliceMax) {
      // the lanes of a group hold the pieces of one token row
#pragma unroll
      for (int d = 1; d < G::kLanes; d <<= 1) smax = fmaxf(smax, __shfl_xor_sync(0xffffffffu, smax, d));
      if (live && sub == 0) e.part_val[(int64_t)(n_warp0 >> 5) * e.part_ld + tok] = smax;
    }
  }
  if (kRes && !OUT_F32 && e.gamma != nullptr) {
    // one sum of squares per token and CTA (128 features): the four warps' shares are added in a fixed order by
    // warp q for tokens 8q .. 8q+7 of the block (ss_red_block: [4 warps][32 tokens], double-buffered by the caller)
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const int q = (n_warp0 >> 5) & 3;
    if (lane < 8) {
      const int tl = q * 8 + lane, tok = tok0 + tl;
      if (tok < tok_limit)
        e.ss_out[(int64_t)tok * e.ss_out_ld + (n_warp0 >> 7)] =
            ((ss_red_block[tl] + ss_red_block[32 + tl]) + ss_red_block[64 + tl]) + ss_red_block[96 + tl];
    }
  }
}

// kEpiArgmax: one 32-token block of a tile.  v: accumulator values (lane = vocabulary id n_warp0 + lane,
// i = token).  After the transpose each lane owns one token and scans its 32 ids in ascending order, so
// the first id among equal logits wins, as torch.argmax / the separate row kernel decide.
__device__ __forceinline__ void epilogue_argmax_block(const float* v, const EpiArgs& e, float* scr, int lane, int n_warp0,
                                                      int tok0, int tok_limit, int N) {
  const bool in_range = n_warp0 + lane < N;
#pragma unroll
  for (int i = 0; i < 32; ++i) scr[i * kScrLd + lane] = in_range ? v[i] : -INFINITY;
  __syncwarp();
  float best = -INFINITY;
  int bj = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float4 f = *reinterpret_cast<const float4*>(scr + lane * kScrLd + 4 * j);
    if (f.x > best) { best = f.x; bj = 4 * j; }
    if (f.y > best) { best = f.y; bj = 4 * j + 1; }
    if (f.z > best) { best = f.z; bj = 4 * j + 2; }
    if (f.w > best) { best = f.w; bj = 4 * j + 3; }
  }
  __syncwarp();  // the scratch is reused by the next block
  const int tok = tok0 + lane;
  // a ragged last weight tile reaches past N: slices that hold no vocabulary id have no slot in the workspace
  if (tok < tok_limit && n_warp0 < N) {
    // one 64-bit word per (slice, token): larger logit first, then the smaller id, under plain unsigned order
    // (-0 and +0 compare equal as floats, so both take +0's key)
    if (best == 0.f) best = 0.f;
    e.part_key[(int64_t)(n_warp0 >> 5) * e.part_ld + tok] =
        ((unsigned long long)rd::float_key(best) << 32) | (unsigned long long)(0xffffffffu - (uint32_t)(n_warp0 + bj));
  }
}

__device__ __forceinline__ float4 ldg_f4(const float* p) {
  float4 r;
  asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "l"(p));
  return r;
}

// Per-token inputs of the rotary epilogue (the position, which leads to the cos/sin rows, and the row of the
// token's slot in the cache), staged in shared memory for the whole tile by the four epilogue warps while the
// tile's main loop still runs.  Fetched inside the block loop they cost ~1.5 k cycles per 32-token block even when
// requested a block ahead: with global loads in flight, the waits for the shared-memory words of the
// transposition waited for them too.
constexpr int kRopeMetaBytes = 2 * kMaxChunk * 4;
constexpr int kEpiStageBytes = 4 * 128 * 16 + 1024;  // residual pieces (8 KB, or the rotary inputs) + the norm's reduction buffer
static_assert(kEpiStageBytes >= kRopeMetaBytes, "staging area");
__device__ __forceinline__ void rope_meta_stage(const EpiArgs& e, int* s_pos, int* s_dst, int tok_base, int tok_limit, int et,
                                                bool is_q, bool is_v) {
#pragma unroll
  for (int t = et; t < kMaxChunk; t += 128) {
    const int tok = tok_base + t;
    if (tok < tok_limit) {
      if (!is_v) {
        const int ps = e.tok_pos[tok];
        s_pos[t] = ps < 0 ? 0 : (ps >= e.n_pos ? e.n_pos - 1 : ps);
      }
      // K and V heads: (row * nkv) * max_len + slot; kv head * max_len is added by the user
      if (!is_q) s_dst[t] = e.tok_row[tok] * e.nkv * e.max_len + e.tok_slot[tok];
    }
  }
}

// Consumer side of the folded RMS norm: the row scales of the tile's tokens, formed once per tile by the four
// epilogue warps (token per thread, the slices of a token added in ascending order) while the main loop runs.
__device__ __forceinline__ void norm_scale_stage(const EpiArgs& e, float* s_scale, int tok_base, int tok_limit, int et) {
#pragma unroll
  for (int t = et; t < kMaxChunk; t += 128) {
    const int tok = tok_base + t;
    if (tok < tok_limit) {
      // a token's slices lie side by side (16-byte aligned rows): few, wide, independent loads
      const float4* src = reinterpret_cast<const float4*>(e.ss_in + (int64_t)tok * e.ss_in_ld);
      float sum = 0.f;
#pragma unroll 8
      for (int q4 = 0; q4 < (e.ss_slices >> 2); ++q4) {
        const float4 f = src[q4];
        sum += f.x;
        sum += f.y;
        sum += f.z;
        sum += f.w;
      }
      for (int sl = e.ss_slices & ~3; sl < e.ss_slices; ++sl) sum += e.ss_in[(int64_t)tok * e.ss_in_ld + sl];
      s_scale[t] = 1.0f / sqrtf(sum / e.norm_dim + e.norm_eps);
    }
  }
}

// Epilogue block of the QKV projection with fused rotary embedding (head_dim 128 = one CTA's 128
// weight rows = one head).  v: this lane's feature d = 32*quarter + lane for the block's 32 tokens.
// The rotation pairs feature d with d +- 64, which lives in the warp two quarters away, so the four
// epilogue warps exchange their transposed blocks through the scratch and meet at a named barrier.
// Values are rounded to bf16 first, as a separate projection would have stored them, so the result
// equals projection -> rope bit for bit.  After the exchange four lanes share a token row (8 features
// each), so the cos/sin reads and the stores of an instruction cover 8 rows, not 32.
__device__ __forceinline__ void epilogue_rope_block(const float* v, const EpiArgs& e, float* scr_all, int quarter, int lane,
                                                    int head, int tok0, int tok_limit, const int* s_pos, const int* s_dst,
                                                    const float* s_scale) {
  float* scr = scr_all + quarter * 32 * kScrLd;
  const bool is_v = head >= e.nh + e.nkv;
  const int sub = lane & 3, row0 = lane >> 2;
  const int d0 = quarter * 32 + sub * 8;
  const float sign = quarter < 2 ? -1.0f : 1.0f;  // rotate_half: (-x2, x1)
  // the cos/sin rows of the block's tokens are requested first (volatile asm keeps them here): their latency
  // runs under the transposition and the exchange below
  float4 cs[4][4];
  if (!is_v) {
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      if (tok0 + row0 + 8 * p < tok_limit) {
        const int pos = s_pos[row0 + 8 * p];
        const float* c = e.cos_t + (int64_t)pos * 128 + d0;
        const float* sn = e.sin_t + (int64_t)pos * 128 + d0;
        cs[p][0] = ldg_f4(c), cs[p][1] = ldg_f4(c + 4), cs[p][2] = ldg_f4(sn), cs[p][3] = ldg_f4(sn + 4);
      }
    }
  }
  if (s_scale != nullptr) {
    // folded RMS norm: the projection of the normalised row is the projection of the row times its scale; scaled and
    // rounded after the exchange, where a lane holds one token's values
#pragma unroll
    for (int i = 0; i < 32; ++i) scr[i * kScrLd + lane] = v[i];
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) scr[i * kScrLd + lane] = __bfloat162float(__float2bfloat16_rn(v[i]));
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");
  float o[4][8];
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const int r = row0 + 8 * p;
    const float* own = scr + r * kScrLd + sub * 8;
    const float4 a0 = *reinterpret_cast<const float4*>(own), a1 = *reinterpret_cast<const float4*>(own + 4);
    o[p][0] = a0.x, o[p][1] = a0.y, o[p][2] = a0.z, o[p][3] = a0.w;
    o[p][4] = a1.x, o[p][5] = a1.y, o[p][6] = a1.z, o[p][7] = a1.w;
    const float sc = s_scale != nullptr ? s_scale[r] : 1.0f;
    if (s_scale != nullptr) {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[p][j] = __bfloat162float(__float2bfloat16_rn(o[p][j] * sc));
    }
    if (!is_v) {
      const float* oth = scr_all + (quarter ^ 2) * 32 * kScrLd + r * kScrLd + sub * 8;
      float4 b0 = *reinterpret_cast<const float4*>(oth), b1 = *reinterpret_cast<const float4*>(oth + 4);
      if (s_scale != nullptr) {
        b0.x = __bfloat162float(__float2bfloat16_rn(b0.x * sc)), b0.y = __bfloat162float(__float2bfloat16_rn(b0.y * sc));
        b0.z = __bfloat162float(__float2bfloat16_rn(b0.z * sc)), b0.w = __bfloat162float(__float2bfloat16_rn(b0.w * sc));
        b1.x = __bfloat162float(__float2bfloat16_rn(b1.x * sc)), b1.y = __bfloat162float(__float2bfloat16_rn(b1.y * sc));
        b1.z = __bfloat162float(__float2bfloat16_rn(b1.z * sc)), b1.w = __bfloat162float(__float2bfloat16_rn(b1.w * sc));
      }
      if (tok0 + r < tok_limit) {
        const float4 c0 = cs[p][0], c1 = cs[p][1], s0 = cs[p][2], s1 = cs[p][3];
        // two rounded products and one rounded sum, as the separate rope kernel computes them
        o[p][0] = __fadd_rn(__fmul_rn(o[p][0], c0.x), __fmul_rn(sign * b0.x, s0.x));
        o[p][1] = __fadd_rn(__fmul_rn(o[p][1], c0.y), __fmul_rn(sign * b0.y, s0.y));
        o[p][2] = __fadd_rn(__fmul_rn(o[p][2], c0.z), __fmul_rn(sign * b0.z, s0.z));
        o[p][3] = __fadd_rn(__fmul_rn(o[p][3], c0.w), __fmul_rn(sign * b0.w, s0.w));
        o[p][4] = __fadd_rn(__fmul_rn(o[p][4], c1.x), __fmul_rn(sign * b1.x, s1.x));
        o[p][5] = __fadd_rn(__fmul_rn(o[p][5], c1.y), __fmul_rn(sign * b1.y, s1.y));
        o[p][6] = __fadd_rn(__fmul_rn(o[p][6], c1.z), __fmul_rn(sign * b1.z, s1.z));
        o[p][7] = __fadd_rn(__fmul_rn(o[p][7], c1.w), __fmul_rn(sign * b1.w, s1.w));
      }
    }
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");  // all four warps have read before the scratch is reused
  const bool is_q = head < e.nh;
  const int kvh = is_v ? head - e.nh - e.nkv : head - e.nh;
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const int tok = tok0 + row0 + 8 * p;
    if (tok < tok_limit) {
      __nv_bfloat16* dst = is_q ? e.q_out + ((int64_t)tok * e.nh + head) * 128 + d0
                                : (is_v ? e.v_cache : e.k_cache) + ((int64_t)s_dst[row0 + 8 * p] + (int64_t)kvh * e.max_len) * 128 + d0;
      uint4 pk;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
      for (int t = 0; t < 4; ++t) h[t] = __floats2bfloat162_rn(o[p][2 * t], o[p][2 * t + 1]);
      *reinterpret_cast<uint4*>(dst) = pk;
    }
  }
}

struct SmemLayout {
  static constexpr int kStageW = BM * BK * 2;         // 16 KB
  static constexpr int kStageA = kMaxChunk * BK * 2;  // 32 KB: two 128-token boxes back to back
  static constexpr int kStages = 4;
  static constexpr int kScratch = 4 * 32 * kScrLd * 4;  // per-epilogue-warp transpose scratch
  static constexpr int kBytes =
      kStages * (kStageW + kStageA) + kScratch + 1024 /*alignment slack*/ + 256 /*barriers*/ + kEpiStageBytes;
};

template <int EPI, bool OUT_F32>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, EpiArgs epi,
                   int m_max, const int32_t* __restrict__ m_dev, int N, int K, int32_t* status) {
  using L = SmemLayout;
  constexpr int kStages = L::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sW = smem;
  uint8_t* sA = smem + kStages * L::kStageW;
  float* scratch = reinterpret_cast<float*>(smem + kStages * (L::kStageW + L::kStageA));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * (L::kStageW + L::kStageA) + L::kScratch);
  uint64_t* full = bars;                    // [kStages]
  uint64_t* empty = bars + kStages;         // [kStages]
  uint64_t* acc_full = bars + 2 * kStages;  // [2]
  uint64_t* acc_empty = acc_full + 2;       // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // staging area of the epilogue warps: rope_meta_stage (kEpiQkvRope) or the residual pieces (ResidualRegs::request)
  int* s_pos = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(bars) + 256);
  int* s_dst = s_pos + kMaxChunk;
  uint4* res_buf = reinterpret_cast<uint4*>(s_pos) + ((threadIdx.x >> 5) & 3) * 128;  // 2 KB per epilogue warp
  float* s_scale = reinterpret_cast<float*>(s_dst + kMaxChunk);  // folded RMS norm, consumer side: see norm_scale_stage
  float* ss_red = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(s_pos) + 8192);  // producer side: 2 x [4][32] floats

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  rd::pdl_launch_dependents();  // the next kernel may set itself up while this one runs

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(2 * kMaxChunk)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // everything above touched only this CTA's shared memory and TMEM; global memory (the live row
  // count, the activations, the output) is valid once the kernels before this one have finished
  rd::pdl_wait();
  const int M = rd::live_rows(m_dev, m_max);
  RD_TIMING_BEGIN();
  const int w_tiles = (N + BM - 1) / BM;
  const Chunking ch = make_chunking(M, w_tiles, gridDim.x);
  const int total_tiles = M > 0 ? w_tiles * ch.n_chunks : 0;
  const int k_blocks = K / BK;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const int w_tile = tile / ch.n_chunks, ci = tile % ch.n_chunks;
        const int cols = chunk_cols(ch, ci, M);
        const int tok0 = ci * ch.chunk;
        const uint32_t bytes = L::kStageW + (cols > 128 ? 2 : 1) * (128 * BK * 2);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&full[stage], bytes);
          tma_load_2d(sW + stage * L::kStageW, &map_w, &full[stage], kb * BK, w_tile * BM);
          tma_load_2d(sA + stage * L::kStageA, &map_a, &full[stage], kb * BK, tok0);
          if (cols > 128) tma_load_2d(sA + stage * L::kStageA + 128 * BK * 2, &map_a, &full[stage], kb * BK, tok0 + 128);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        if (atomicCAS((int*)abort_flag, 0, 1) == 0 && status) atomicExch(status, 1);
        // let bulk copies that are still in flight land before the CTA's shared memory goes away
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int local = 0;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++local) {
        const int ci = tile % ch.n_chunks;
        const uint32_t idesc = umma_instr_desc(chunk_cols(ch, ci, M));
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kMaxChunk;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t dw = umma_smem_desc(smem_u32(sW + stage * L::kStageW));
          const uint64_t da = umma_smem_desc(smem_u32(sA + stage * L::kStageA));
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // advance the start address by 16 elements = 32 bytes = 2 sixteen-byte units
            umma_f16(d_tmem, dw + 2 * k, da + 2 * k, idesc, (kb | k) != 0);
          }
          umma_commit(&empty[stage]);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&acc_full[acc]);
      }
      if (!ok && atomicCAS((int*)abort_flag, 0, 1) == 0 && status) atomicExch(status, 2);
    }
  } else {
    // ---------------- epilogue warps ----------------
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
    float* scr = scratch + (warp - 2) * 32 * kScrLd;
    constexpr int kOut = (EPI == RD_EPI_SWIGLU) ? 16 : 32;
    constexpr bool kRes = (EPI == RD_EPI_BIAS_SILU_RES || EPI == RD_EPI_RES);
    const int esz = OUT_F32 ? 4 : 2;
    const bool aligned = (((uintptr_t)epi.C | (uintptr_t)(kRes ? epi.R : epi.C)) % 16 == 0) && ((epi.ldc * esz) % 16 == 0) &&
                         (!kRes || (epi.ldr * esz) % 16 == 0);
    bool ok = true;
    int local = 0;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++local) {
      const int w_tile = tile / ch.n_chunks, ci = tile % ch.n_chunks;
      const int cols = chunk_cols(ch, ci, M);
      const int tok_base = ci * ch.chunk;
      // tokens past the chunk belong to the next chunk's tile (its columns here were not computed)
      const int tok_limit = min(M, tok_base + ch.chunk);
      const int n_warp0 = w_tile * BM + quarter * 32;
      const bool vec_ok = aligned && (n_warp0 + 32 <= N);
      const int out0 = (EPI == RD_EPI_SWIGLU) ? (n_warp0 >> 1) : n_warp0;
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      // the first block's residual row is fetched while the main loop of this tile still runs
      ResidualRegs<OUT_F32, kOut> res_next;
      // this lane's bias, read once per tile and ahead of the wait (a load inside the block loop stalls every block)
      constexpr bool kBias = (EPI == RD_EPI_BIAS || EPI == RD_EPI_BIAS_SILU || EPI == RD_EPI_BIAS_SILU_RES);
      const float bias = (kBias && n_warp0 + lane < N) ? __bfloat162float(epi.bias[n_warp0 + lane]) : 0.f;
      const int rope_head = (n_warp0 - quarter * 32) / 128;
      constexpr bool kNormIn = (EPI == kEpiQkvRope || EPI == RD_EPI_SWIGLU);
      const bool norm_in = kNormIn && epi.ss_in != nullptr;
      if (EPI == kEpiQkvRope || norm_in) asm volatile("bar.sync 1, 128;" ::: "memory");  // the tile before has read its entries
      if (EPI == kEpiQkvRope)
        rope_meta_stage(epi, s_pos, s_dst, tok_base, tok_limit, (int)threadIdx.x - 64, rope_head < epi.nh,
                        rope_head >= epi.nh + epi.nkv);
      if (norm_in) norm_scale_stage(epi, s_scale, tok_base, tok_limit, (int)threadIdx.x - 64);
      // producer side of the folded RMS norm: this lane's eight gamma values (its features are the same in every block)
      uint4 gamma8 = make_uint4(0u, 0u, 0u, 0u);
      if (kRes && !OUT_F32 && epi.gamma != nullptr && vec_ok)
        gamma8 = *reinterpret_cast<const uint4*>(epi.gamma + n_warp0 + (lane & 3) * 8);
      if (kRes && vec_ok) {
        if (OUT_F32)
          res_next.load(epi, tok_base, out0, tok_limit, lane);
        else
          res_next.request(epi, tok_base, out0, tok_limit, lane, res_buf, 0u);
      }
      if (!mbar_wait(&acc_full[acc], acc_phase, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (EPI == kEpiQkvRope || norm_in) asm volatile("bar.sync 1, 128;" ::: "memory");  // the staged entries are visible
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kMaxChunk;
#pragma unroll 1
      for (int c = 0; c < cols; c += 32) {
        if (kRes && vec_ok && !OUT_F32) res_next.take(res_buf, lane);
        ResidualRegs<OUT_F32, kOut> res_cur = res_next;
        if (kRes && vec_ok && c + 32 < cols) {
          if (OUT_F32)
            res_next.load(epi, tok_base + c + 32, out0, tok_limit, lane);
          else
            res_next.request(epi, tok_base + c + 32, out0, tok_limit, lane, res_buf, res_cur.q[EpiLanes<OUT_F32, kOut>::kPasses - 1].w);
        }
        uint32_t r[32];
        tmem_ld32(t_row + c, r);
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
        if (EPI == kEpiQkvRope) {
          epilogue_rope_block(v, epi, scratch, quarter, lane, rope_head, tok_base + c, tok_limit, s_pos + c, s_dst + c,
                              norm_in ? s_scale + c : nullptr);
        } else if (EPI == kEpiArgmax) {
          epilogue_argmax_block(v, epi, scr, lane, n_warp0, tok_base + c, tok_limit, N);
        } else {
          epilogue_math<EPI>(v, epi, n_warp0 + lane, N, !vec_ok, bias);
          epilogue_block<EPI, OUT_F32>(v, epi, scr, lane, n_warp0, tok_base + c, tok_limit, N, vec_ok, res_cur,
                                       norm_in ? s_scale + c : nullptr, gamma8, ss_red + ((c >> 5) & 1) * 128);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
    }
    if (!ok && lane == 0 && atomicCAS((int*)abort_flag, 0, 1) == 0 && status) atomicExch(status, 3);
  }

  tc_fence_before();
  __syncthreads();
  RD_TIMING_END(M, N, K);
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * kMaxChunk) : "memory");
  }
}


// =================================================================================================
// CTA-pair variant (cta_group::2): two CTAs of a cluster share one MMA of M = 256 weight rows.
// Each CTA stages its own 128 weight rows and HALF of the token tile, so the shared-memory traffic
// per MMA drops by a third and the per-CTA L2 traffic by the same; the leader CTA's elected thread
// issues the MMAs for both, each CTA's TMEM receives its 128 rows of the accumulator, and each
// CTA's epilogue warps store their own rows.  Signalling: both CTAs' bulk loads complete on the
// LEADER's full barrier; the leader frees a stage and publishes an accumulator with one
// tcgen05.commit that arrives on the barrier of both CTAs (the bulk loads themselves are never
// multicast); the peer's epilogue warps release the accumulator with remote arrives on the
// leader's barrier.

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t mapa_u32(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t leader_bar_cluster_addr, int c0,
                                                 int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::
          "r"(smem_u32(dst)),
      "l"(map), "r"(leader_bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc)
      : "memory");
}
// One commit that arrives on the barrier at the same shared-memory offset in every CTA of `cta_mask`
// (both CTAs of the pair): half the commit instructions of two plain commits, and commits are not free.
__device__ __forceinline__ void umma_commit_pair_both(uint64_t* bar) {
  const uint16_t cta_mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(cta_mask)
      : "memory");
}
__device__ __forceinline__ uint32_t umma_instr_desc_pair(int n) {
  // fp32 accumulator, bf16 A and B, both K-major, M = 256 over the CTA pair, N = n
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

constexpr int kTokBoxBytes = kTokBox * BK * 2;  // 4 KB
struct SmemLayoutPair {
  static constexpr int kSub = 1;                       // k-blocks of 64 per pipeline stage (2 with 3 stages measured the same)
  static constexpr int kBoxW = BM * BK * 2;            // 16 KB: this CTA's 128 weight rows of one k-block
  static constexpr int kBoxA = 128 * BK * 2;           // 16 KB: this CTA's half of the token tile of one k-block (up to 4 boxes)
  static constexpr int kStageW = kSub * kBoxW;
  static constexpr int kStageA = kSub * kBoxA;
  static constexpr int kStages = 6;
  static constexpr int kScratch = 4 * 32 * kScrLd * 4;
  static constexpr int kBytes = kStages * (kStageW + kStageA) + kScratch + 1024 + 256 + kEpiStageBytes;
};

template <int EPI, bool OUT_F32>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_tc_pair_kernel(const __grid_constant__ TokMaps maps_a, const __grid_constant__ CUtensorMap map_w, EpiArgs epi,
                        int m_max, const int32_t* __restrict__ m_dev, int N, int K, int32_t* status) {
  using L = SmemLayoutPair;
  constexpr int kStages = L::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sW = smem;
  uint8_t* sA = smem + kStages * L::kStageW;
  float* scratch = reinterpret_cast<float*>(smem + kStages * (L::kStageW + L::kStageA));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * (L::kStageW + L::kStageA) + L::kScratch);
  uint64_t* full = bars;                    // [kStages] used in the leader CTA
  uint64_t* empty = bars + kStages;         // [kStages] one per CTA
  uint64_t* acc_full = bars + 2 * kStages;  // [2] one per CTA
  uint64_t* acc_empty = acc_full + 2;       // [2] used in the leader CTA (8 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // staging area of the epilogue warps: rope_meta_stage (kEpiQkvRope) or the residual pieces (ResidualRegs::request)
  int* s_pos = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(bars) + 256);
  int* s_dst = s_pos + kMaxChunk;
  uint4* res_buf = reinterpret_cast<uint4*>(s_pos) + ((threadIdx.x >> 5) & 3) * 128;  // 2 KB per epilogue warp
  float* s_scale = reinterpret_cast<float*>(s_dst + kMaxChunk);  // folded RMS norm, consumer side: see norm_scale_stage
  float* ss_red = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(s_pos) + 8192);  // producer side: 2 x [4][32] floats

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  rd::pdl_launch_dependents();  // the next kernel may set itself up while this one runs
  if (threadIdx.x == 0) {
    // the descriptors are kernel parameters: their fetch may start before the dependency wait
    for (int i = 0; i < 4; ++i) asm volatile("prefetch.tensormap [%0];" ::"l"(&maps_a.m[i]) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 8);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(2 * kMaxChunk)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  rd::pdl_wait();  // global memory is valid once the kernels before this one have finished
  const int M = rd::live_rows(m_dev, m_max);
  RD_TIMING_BEGIN();
  const int w_pairs = (N + 2 * BM - 1) / (2 * BM);
  const Chunking ch = make_chunking(M, w_pairs, n_pairs);
  const int all_tiles = M > 0 ? w_pairs * ch.n_chunks : 0;
  const int k_blocks = K / BK;
  // The launch lasts rounds = ceil(tiles / pairs) tile times however the tiles are dealt, so only as many
  // pairs take part as fill those rounds evenly (258 tiles on 74 pairs: 4 rounds, 65 pairs); the others
  // leave at once, and the SMs they free lower the power the busy ones share (c2 step 12.99 -> 12.97 ms).
  int n_active = n_pairs;
  if (all_tiles > 0) {
    const int rounds = (all_tiles + n_pairs - 1) / n_pairs;
    n_active = (all_tiles + rounds - 1) / rounds;
  }
  const int total_tiles = pair_id < n_active ? all_tiles : 0;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair_id; ok && tile < total_tiles; tile += n_active) {
        const int w_pair = tile / ch.n_chunks, ci = tile % ch.n_chunks;
        const int cols = chunk_cols(ch, ci, M);
        const int tok0 = ci * ch.chunk + (int)rank * (cols >> 1);  // this CTA's half of the chunk
        const int n_box = ((cols >> 1) + kTokBox - 1) / kTokBox;
        const CUtensorMap* map_a = &maps_a.m[n_box - 1];
        const int w_row0 = w_pair * 2 * BM + (int)rank * BM;
        for (int kb = 0; kb < k_blocks; kb += L::kSub) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) {
            ok = false;
            break;
          }
          const int n_sub = min(L::kSub, k_blocks - kb);
          const uint32_t leader_full = mapa_u32(smem_u32(&full[stage]), 0);
          if (rank == 0) mbar_expect_tx(&full[stage], 2 * n_sub * (L::kBoxW + n_box * kTokBoxBytes));
          for (int sb = 0; sb < n_sub; ++sb) {
            tma_load_2d_pair(sW + stage * L::kStageW + sb * L::kBoxW, &map_w, leader_full, (kb + sb) * BK, w_row0);
            // one box of just the rows the chunk's half fills (rounded up to 32): a chunk of 192 tokens moves 96
            // rows per CTA, not 128 (1-2 % on the projections with four chunks).  Several 32-row boxes instead of
            // one tall one made the loop 25 % slower: the cost of a load is per box far more than per byte.
            tma_load_2d_pair(sA + stage * L::kStageA + sb * L::kBoxA, map_a, leader_full, (kb + sb) * BK, tok0);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        if (atomicCAS((int*)abort_flag, 0, 1) == 0 && status) atomicExch(status, 11);
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (lane == 0 && rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int local = 0;
      for (int tile = pair_id; ok && tile < total_tiles; tile += n_active, ++local) {
        const int ci = tile % ch.n_chunks;
        const uint32_t idesc = umma_instr_desc_pair(chunk_cols(ch, ci, M));
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kMaxChunk;
        for (int kb = 0; kb < k_blocks; kb += L::kSub) {
          if (!mbar_wait(&full[stage], phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const int n_sub = min(L::kSub, k_blocks - kb);
          for (int sb = 0; sb < n_sub; ++sb) {
            const uint64_t dw = umma_smem_desc(smem_u32(sW + stage * L::kStageW + sb * L::kBoxW));
            const uint64_t da = umma_smem_desc(smem_u32(sA + stage * L::kStageA + sb * L::kBoxA));
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) umma_f16_pair(d_tmem, dw + 2 * k, da + 2 * k, idesc, (kb | sb | k) != 0);
          }
          umma_commit_pair_both(&empty[stage]);  // frees the stage in both CTAs
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) {
          umma_commit_pair_both(&acc_full[acc]);
        }
      }
      if (!ok && atomicCAS((int*)abort_flag, 0, 1) == 0 && status) atomicExch(status, 12);
    }
  } else {
    // ---------------- epilogue warps (both CTAs, own 128 weight rows) ----------------
    const int quarter = warp & 3;
    float* scr = scratch + (warp - 2) * 32 * kScrLd;
    constexpr int kOut = (EPI == RD_EPI_SWIGLU) ? 16 : 32;
    constexpr bool kRes = (EPI == RD_EPI_BIAS_SILU_RES || EPI == RD_EPI_RES);
    const int esz = OUT_F32 ? 4 : 2;
    const bool aligned = (((uintptr_t)epi.C | (uintptr_t)(kRes ? epi.R : epi.C)) % 16 == 0) && ((epi.ldc * esz) % 16 == 0) &&
                         (!kRes || (epi.ldr * esz) % 16 == 0);
    bool ok = true;
    int local = 0;
    for (int tile = pair_id; ok && tile < total_tiles; tile += n_active, ++local) {
      const int w_pair = tile / ch.n_chunks, ci = tile % ch.n_chunks;
      const int cols = chunk_cols(ch, ci, M);
      const int tok_base = ci * ch.chunk;
      const int tok_limit = min(M, tok_base + ch.chunk);
      const int n_warp0 = w_pair * 2 * BM + (int)rank * BM + quarter * 32;
      const bool vec_ok = aligned && (n_warp0 + 32 <= N);
      const int out0 = (EPI == RD_EPI_SWIGLU) ? (n_warp0 >> 1) : n_warp0;
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      ResidualRegs<OUT_F32, kOut> res_next;
      // this lane's bias, read once per tile and ahead of the wait (a load inside the block loop stalls every block)
      constexpr bool kBias = (EPI == RD_EPI_BIAS || EPI == RD_EPI_BIAS_SILU || EPI == RD_EPI_BIAS_SILU_RES);
      const float bias = (kBias && n_warp0 + lane < N) ? __bfloat162float(epi.bias[n_warp0 + lane]) : 0.f;
      const int rope_head = (n_warp0 - quarter * 32) / 128;
      constexpr bool kNormIn = (EPI == kEpiQkvRope || EPI == RD_EPI_SWIGLU);
      const bool norm_in = kNormIn && epi.ss_in != nullptr;
      if (EPI == kEpiQkvRope || norm_in) asm volatile("bar.sync 1, 128;" ::: "memory");  // the tile before has read its entries
      if (EPI == kEpiQkvRope)
        rope_meta_stage(epi, s_pos, s_dst, tok_base, tok_limit, (int)threadIdx.x - 64, rope_head < epi.nh,
                        rope_head >= epi.nh + epi.nkv);
      if (norm_in) norm_scale_stage(epi, s_scale, tok_base, tok_limit, (int)threadIdx.x - 64);
      // producer side of the folded RMS norm: this lane's eight gamma values (its features are the same in every block)
      uint4 gamma8 = make_uint4(0u, 0u, 0u, 0u);
      if (kRes && !OUT_F32 && epi.gamma != nullptr && vec_ok)
        gamma8 = *reinterpret_cast<const uint4*>(epi.gamma + n_warp0 + (lane & 3) * 8);
      if (kRes && vec_ok) {
        if (OUT_F32)
          res_next.load(epi, tok_base, out0, tok_limit, lane);
        else
          res_next.request(epi, tok_base, out0, tok_limit, lane, res_buf, 0u);
      }
      if (!mbar_wait(&acc_full[acc], acc_phase, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (EPI == kEpiQkvRope || norm_in) asm volatile("bar.sync 1, 128;" ::: "memory");  // the staged entries are visible
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kMaxChunk;
#pragma unroll 1
      for (int c = 0; c < cols; c += 32) {
        if (kRes && vec_ok && !OUT_F32) res_next.take(res_buf, lane);
        ResidualRegs<OUT_F32, kOut> res_cur = res_next;
        if (kRes && vec_ok && c + 32 < cols) {
          if (OUT_F32)
            res_next.load(epi, tok_base + c + 32, out0, tok_limit, lane);
          else
            res_next.request(epi, tok_base + c + 32, out0, tok_limit, lane, res_buf, res_cur.q[EpiLanes<OUT_F32, kOut>::kPasses - 1].w);
        }
        uint32_t r[32];
        tmem_ld32(t_row + c, r);
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
        if (EPI == kEpiQkvRope) {
          epilogue_rope_block(v, epi, scratch, quarter, lane, rope_head, tok_base + c, tok_limit, s_pos + c, s_dst + c,
                              norm_in ? s_scale + c : nullptr);
        } else if (EPI == kEpiArgmax) {
          epilogue_argmax_block(v, epi, scr, lane, n_warp0, tok_base + c, tok_limit, N);
        } else {
          epilogue_math<EPI>(v, epi, n_warp0 + lane, N, !vec_ok, bias);
          epilogue_block<EPI, OUT_F32>(v, epi, scr, lane, n_warp0, tok_base + c, tok_limit, N, vec_ok, res_cur,
                                       norm_in ? s_scale + c : nullptr, gamma8, ss_red + ((c >> 5) & 1) * 128);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&acc_empty[acc]), 0));
    }
    if (!ok && lane == 0 && atomicCAS((int*)abort_flag, 0, 1) == 0 && status) atomicExch(status, 13);
  }

  // Neither CTA may leave (or free TMEM) while its peer can still signal its barriers or while
  // MMAs of the pair are in flight: meet at a cluster barrier first.
  tc_fence_before();
  __syncthreads();
  RD_TIMING_END(M, N, K);
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * kMaxChunk) : "memory");
  }
}

// Second half of the fused LM-head argmax: the partial results are 64-bit keys whose unsigned order is
// (logit descending, id ascending), so the merge is a plain maximum.  A block serves 8 tokens with 32
// groups of threads walking the slices (each 32-byte sector of the [slice][token] array is read once).
constexpr int kMergeTok = 8, kMergeGroups = 32;
__global__ void __launch_bounds__(kMergeTok* kMergeGroups) argmax_merge_kernel(const unsigned long long* __restrict__ part_key, int64_t ld,
                                                                              int n_slices, int m_max,
                                                                              const int32_t* __restrict__ m_dev,
                                                                              int32_t* __restrict__ out32, int64_t* __restrict__ out64) {
  rd::pdl_launch_dependents();
  rd::pdl_wait();
  const int M = rd::live_rows(m_dev, m_max);
  if ((int)blockIdx.x * kMergeTok >= M) return;
  const int t = threadIdx.x % kMergeTok, g = threadIdx.x / kMergeTok;
  const int tok = blockIdx.x * kMergeTok + t;
  unsigned long long best = 0ull;
  if (tok < M) {
#pragma unroll 4
    for (int sl = g; sl < n_slices; sl += kMergeGroups) {
      const unsigned long long k = part_key[(int64_t)sl * ld + tok];
      best = k > best ? k : best;
    }
  }
  __shared__ unsigned long long sk[kMergeGroups][kMergeTok];
  sk[g][t] = best;
  __syncthreads();
  if (g == 0 && tok < M) {
#pragma unroll
    for (int o = 1; o < kMergeGroups; ++o) best = sk[o][t] > best ? sk[o][t] : best;
    const int id = (int)(0xffffffffu - (uint32_t)(best & 0xffffffffull));
    if (out32) out32[tok] = id;
    if (out64) out64[tok] = id;
  }
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

bool make_map(CUtensorMap* map, const void* base, int64_t ld_elems, int rows, int cols, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld_elems * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename Kern>
int launch_cluster2(Kern kern, int grid, int smem_bytes, cudaStream_t s, const GemmPlan* p, const EpiArgs& e, const int32_t* m_dev,
                    int32_t* status) {
  // the attribute is set once per kernel (this template is shared by every kernel of the same signature), so that
  // steady-state launches are pure launches
  static const void* configured[64];
  static int n_configured = 0;
  bool seen = false;
  for (int i = 0; i < n_configured; ++i) seen = seen || configured[i] == (const void*)kern;
  if (!seen) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (n_configured < 64) configured[n_configured++] = (const void*)kern;
  }
  cudaError_t err = rd::launch_chained(kern, dim3(grid), dim3(kThreads), smem_bytes, s, 2, p->maps_a, p->map_w, e, p->m_max, m_dev,
                                       p->N, p->K, status);
  RD_CHECK_CHAINED(err);
  return RD_OK;
}

template <int EPI>
int launch_out(const GemmPlan* p, int out_dtype, const EpiArgs& e, const int32_t* m_dev, int32_t* status, cudaStream_t s) {
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) sm_count = 148;
  }
  // upper bound of the tile count with the finest chunking the kernel may choose (64 tokens)
  const int chunks = (p->m_max + 63) / 64;
  if (p->N >= 2 * BM && g_use_pairs) {
    // CTA pairs: one pair per 256 weight rows x token chunk
    const int tiles = chunks * ((p->N + 2 * BM - 1) / (2 * BM));
    const int max_pairs = sm_count / 2;
    const int grid = 2 * (tiles < max_pairs ? tiles : max_pairs);
    int rc;
    if (out_dtype == RD_F32)
      rc = launch_cluster2(gemm_tc_pair_kernel<EPI, true>, grid, SmemLayoutPair::kBytes, s, p, e, m_dev, status);
    else
      rc = launch_cluster2(gemm_tc_pair_kernel<EPI, false>, grid, SmemLayoutPair::kBytes, s, p, e, m_dev, status);
    if (rc != RD_OK) return rc;
    RD_CHECK_LAUNCH();
    return RD_OK;
  }
  using L = SmemLayout;
  const int tiles = chunks * ((p->N + BM - 1) / BM);
  const int grid = tiles < sm_count ? tiles : sm_count;
  if (out_dtype == RD_F32) {
    auto kern = gemm_tc_kernel<EPI, true>;
    static bool smem_set = false;
    if (!smem_set) {
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes);
      smem_set = true;
    }
    if (rd::launch_chained(kern, dim3(grid), dim3(kThreads), L::kBytes, s, 1, p->map_a, p->map_w, e, p->m_max, m_dev, p->N, p->K,
                           status) != cudaSuccess)
      return RD_ERR_LAUNCH;
  } else {
    auto kern = gemm_tc_kernel<EPI, false>;
    static bool smem_set = false;
    if (!smem_set) {
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes);
      smem_set = true;
    }
    if (rd::launch_chained(kern, dim3(grid), dim3(kThreads), L::kBytes, s, 1, p->map_a, p->map_w, e, p->m_max, m_dev, p->N, p->K,
                           status) != cudaSuccess)
      return RD_ERR_LAUNCH;
  }
  RD_CHECK_LAUNCH();
  return RD_OK;
}

int launch_epi(const GemmPlan* p, int out_dtype, const EpiArgs& e, const int32_t* m_dev, int epilogue, int32_t* status,
               cudaStream_t s) {
  switch (epilogue) {
    case RD_EPI_NONE: return launch_out<RD_EPI_NONE>(p, out_dtype, e, m_dev, status, s);
    case RD_EPI_BIAS: return launch_out<RD_EPI_BIAS>(p, out_dtype, e, m_dev, status, s);
    case RD_EPI_BIAS_SILU: return launch_out<RD_EPI_BIAS_SILU>(p, out_dtype, e, m_dev, status, s);
    case RD_EPI_BIAS_SILU_RES: return launch_out<RD_EPI_BIAS_SILU_RES>(p, out_dtype, e, m_dev, status, s);
    case RD_EPI_RES: return launch_out<RD_EPI_RES>(p, out_dtype, e, m_dev, status, s);
    case RD_EPI_SWIGLU: return launch_out<RD_EPI_SWIGLU>(p, out_dtype, e, m_dev, status, s);
    case kEpiQkvRope: return launch_out<kEpiQkvRope>(p, out_dtype, e, m_dev, status, s);
    case kEpiArgmax: return launch_out<kEpiArgmax>(p, out_dtype, e, m_dev, status, s);
    case kEpiSliceMax: return launch_out<kEpiSliceMax>(p, out_dtype, e, m_dev, status, s);
    default: return RD_ERR_ARG;
  }
}

}  // namespace

extern "C" void* rd_gemm_plan_create(const void* A, int64_t lda, int m_max, const void* W, int64_t ldw, int N, int K) {
  if (!A || !W || m_max < 1 || N < 1 || K < BK || K % BK != 0 || lda < K || ldw < K) return nullptr;
  if (((uintptr_t)A & 15) || ((uintptr_t)W & 15) || (lda * 2) % 16 || (ldw * 2) % 16) return nullptr;
  GemmPlan* p = new GemmPlan();
  p->m_max = m_max;
  p->N = N;
  p->K = K;
  bool ok = make_map(&p->map_a, A, lda, m_max, K, 128) && make_map(&p->map_w, W, ldw, N, K, BM);
  for (int i = 0; ok && i < 4; ++i) ok = make_map(&p->maps_a.m[i], A, lda, m_max, K, (i + 1) * kTokBox);
  if (!ok) {
    delete p;
    return nullptr;
  }
  return p;
}

extern "C" void rd_gemm_plan_destroy(void* plan) { delete static_cast<GemmPlan*>(plan); }

extern "C" int rd_gemm_bf16_tc(const void* plan, int out_dtype, void* C, int64_t ldc, const void* bias, const void* R,
                               int64_t ldr, const int32_t* m_dev, int epilogue, int32_t* status, void* stream) {
  RD_REQUIRE(plan && C, RD_ERR_ARG);
  RD_REQUIRE(out_dtype == RD_F32 || out_dtype == RD_BF16, RD_ERR_DTYPE);
  const GemmPlan* p = static_cast<const GemmPlan*>(plan);
  const bool need_bias = epilogue == RD_EPI_BIAS || epilogue == RD_EPI_BIAS_SILU || epilogue == RD_EPI_BIAS_SILU_RES;
  const bool need_res = epilogue == RD_EPI_BIAS_SILU_RES || epilogue == RD_EPI_RES;
  RD_REQUIRE(!need_bias || bias, RD_ERR_ARG);
  RD_REQUIRE(!need_res || R, RD_ERR_ARG);
  RD_REQUIRE(epilogue != RD_EPI_SWIGLU || p->N % 2 == 0, RD_ERR_SIZE);
  EpiArgs e{};
  e.C = C;
  e.ldc = ldc;
  e.bias = (const __nv_bfloat16*)bias;
  e.R = R;
  e.ldr = ldr;
  cudaStream_t s = (cudaStream_t)stream;
  return launch_epi(p, out_dtype, e, m_dev, epilogue, status, s);
}

static bool norm_in_ok(const GemmPlan* p, const float* ss_in, int64_t ss_ld, int ss_slices, int norm_dim, float eps) {
  (void)p;
  return ss_in && ((uintptr_t)ss_in & 15) == 0 && ss_slices >= 1 && ss_ld >= ss_slices && ss_ld % 4 == 0 && norm_dim >= 1 &&
         eps >= 0.f;
}

extern "C" int rd_gemm_bf16_tc_res_norm(const void* plan, void* C, int64_t ldc, const void* R, int64_t ldr, const int32_t* m_dev,
                                        const void* gamma, void* C2, int64_t ldc2, float* ss_out, int64_t ss_ld,
                                        int32_t* status, void* stream) {
  RD_REQUIRE(plan && C && R && gamma && C2 && ss_out, RD_ERR_ARG);
  const GemmPlan* p = static_cast<const GemmPlan*>(plan);
  RD_REQUIRE(p->N % 128 == 0 && ss_ld >= p->N / 128, RD_ERR_SIZE);
  RD_REQUIRE((((uintptr_t)C | (uintptr_t)R | (uintptr_t)gamma | (uintptr_t)C2) & 15) == 0 && (ldc * 2) % 16 == 0 &&
                 (ldr * 2) % 16 == 0 && (ldc2 * 2) % 16 == 0,
             RD_ERR_ALIGN);
  EpiArgs e{};
  e.C = C;
  e.ldc = ldc;
  e.R = R;
  e.ldr = ldr;
  e.gamma = (const __nv_bfloat16*)gamma;
  e.C2 = (__nv_bfloat16*)C2;
  e.ldc2 = ldc2;
  e.ss_out = ss_out;
  e.ss_out_ld = ss_ld;
  return launch_epi(p, RD_BF16, e, m_dev, RD_EPI_RES, status, (cudaStream_t)stream);
}

extern "C" int rd_gemm_bf16_tc_swiglu_normed(const void* plan, void* C, int64_t ldc, const int32_t* m_dev, const float* ss_in,
                                             int64_t ss_ld, int ss_slices, int norm_dim, float eps, int32_t* status,
                                             void* stream) {
  RD_REQUIRE(plan && C, RD_ERR_ARG);
  const GemmPlan* p = static_cast<const GemmPlan*>(plan);
  RD_REQUIRE(p->N % 2 == 0 && norm_in_ok(p, ss_in, ss_ld, ss_slices, norm_dim, eps), RD_ERR_SIZE);
  EpiArgs e{};
  e.C = C;
  e.ldc = ldc;
  e.ss_in = ss_in;
  e.ss_in_ld = ss_ld;
  e.ss_slices = ss_slices;
  e.norm_dim = (float)norm_dim;
  e.norm_eps = eps;
  return launch_epi(p, RD_BF16, e, m_dev, RD_EPI_SWIGLU, status, (cudaStream_t)stream);
}

static int qkv_rope_launch(const void* plan, const int32_t* m_dev, void* q_out, void* k_cache, void* v_cache,
                           const int32_t* tok_row, const int32_t* tok_pos, const int32_t* tok_slot, const float* cos_table,
                           const float* sin_table, int n_pos, int nh, int nkv, int hd, int max_len, const float* ss_in,
                           int64_t ss_ld, int ss_slices, int norm_dim, float eps, int32_t* status, void* stream) {
  RD_REQUIRE(plan && q_out && k_cache && v_cache && tok_row && tok_pos && tok_slot && cos_table && sin_table, RD_ERR_ARG);
  const GemmPlan* p = static_cast<const GemmPlan*>(plan);
  RD_REQUIRE(hd == 128 && nh >= 1 && nkv >= 1 && n_pos >= 1 && max_len >= 1, RD_ERR_SIZE);
  RD_REQUIRE(p->N == (nh + 2 * nkv) * hd, RD_ERR_SIZE);
  RD_REQUIRE((((uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)cos_table | (uintptr_t)sin_table) & 15) == 0,
             RD_ERR_ALIGN);
  EpiArgs e{};
  e.C = q_out;  // unused by this epilogue; kept non-null for the common alignment checks in the kernel
  e.ldc = (int64_t)nh * hd;
  e.q_out = (__nv_bfloat16*)q_out;
  e.k_cache = (__nv_bfloat16*)k_cache;
  e.v_cache = (__nv_bfloat16*)v_cache;
  e.tok_row = tok_row;
  e.tok_pos = tok_pos;
  e.tok_slot = tok_slot;
  e.cos_t = cos_table;
  e.sin_t = sin_table;
  e.n_pos = n_pos;
  e.nh = nh;
  e.nkv = nkv;
  e.max_len = max_len;
  if (ss_in) {
    RD_REQUIRE(norm_in_ok(p, ss_in, ss_ld, ss_slices, norm_dim, eps), RD_ERR_SIZE);
    e.ss_in = ss_in;
    e.ss_in_ld = ss_ld;
    e.ss_slices = ss_slices;
    e.norm_dim = (float)norm_dim;
    e.norm_eps = eps;
  }
  return launch_epi(p, RD_BF16, e, m_dev, kEpiQkvRope, status, (cudaStream_t)stream);
}

extern "C" int rd_gemm_bf16_tc_qkv_rope(const void* plan, const int32_t* m_dev, void* q_out, void* k_cache, void* v_cache,
                                        const int32_t* tok_row, const int32_t* tok_pos, const int32_t* tok_slot,
                                        const float* cos_table, const float* sin_table, int n_pos, int nh, int nkv, int hd,
                                        int max_len, int32_t* status, void* stream) {
  return qkv_rope_launch(plan, m_dev, q_out, k_cache, v_cache, tok_row, tok_pos, tok_slot, cos_table, sin_table, n_pos, nh, nkv,
                         hd, max_len, nullptr, 0, 0, 0, 0.f, status, stream);
}

extern "C" int rd_gemm_bf16_tc_qkv_rope_normed(const void* plan, const int32_t* m_dev, void* q_out, void* k_cache, void* v_cache,
                                               const int32_t* tok_row, const int32_t* tok_pos, const int32_t* tok_slot,
                                               const float* cos_table, const float* sin_table, int n_pos, int nh, int nkv,
                                               int hd, int max_len, const float* ss_in, int64_t ss_ld, int ss_slices,
                                               int norm_dim, float eps, int32_t* status, void* stream) {
  RD_REQUIRE(ss_in, RD_ERR_ARG);
  return qkv_rope_launch(plan, m_dev, q_out, k_cache, v_cache, tok_row, tok_pos, tok_slot, cos_table, sin_table, n_pos, nh, nkv,
                         hd, max_len, ss_in, ss_ld, ss_slices, norm_dim, eps, status, stream);
}

static inline int64_t part_ld_of(int m_max) { return ((int64_t)m_max + 31) / 32 * 32; }

extern "C" int64_t rd_gemm_argmax_workspace_bytes(int m_max, int N) {
  if (m_max < 1 || N < 1) return 0;
  return (int64_t)((N + 31) / 32) * part_ld_of(m_max) * 8;
}

extern "C" int rd_gemm_bf16_tc_argmax(const void* plan, const int32_t* m_dev, void* workspace, int64_t workspace_bytes,
                                      int32_t* out32, int64_t* out64, int32_t* status, void* stream) {
  RD_REQUIRE(plan && workspace && (out32 || out64), RD_ERR_ARG);
  const GemmPlan* p = static_cast<const GemmPlan*>(plan);
  RD_REQUIRE(((uintptr_t)workspace & 15) == 0, RD_ERR_ALIGN);
  RD_REQUIRE(workspace_bytes >= rd_gemm_argmax_workspace_bytes(p->m_max, p->N), RD_ERR_CAPACITY);
  const int n_slices = (p->N + 31) / 32;
  const int64_t ld = part_ld_of(p->m_max);
  EpiArgs e{};
  e.part_key = (unsigned long long*)workspace;
  e.part_ld = ld;
  e.C = workspace;  // no output matrix; kept non-null and aligned for the checks the epilogues share
  e.ldc = 4;
  cudaStream_t s = (cudaStream_t)stream;
  int rc = launch_epi(p, RD_F32, e, m_dev, kEpiArgmax, status, s);
  if (rc != RD_OK) return rc;
  cudaError_t err = rd::launch_chained(argmax_merge_kernel, dim3((p->m_max + kMergeTok - 1) / kMergeTok), dim3(kMergeTok * kMergeGroups), 0,
                                       s, 1, (const unsigned long long*)e.part_key, ld, n_slices, p->m_max, m_dev, out32, out64);
  RD_CHECK_CHAINED(err);
  return RD_OK;
}

extern "C" int rd_gemm_bf16_tc_slicemax(const void* plan, int out_dtype, void* C, int64_t ldc, const int32_t* m_dev,
                                        float* slice_max, int64_t slice_ld, int32_t* status, void* stream) {
  RD_REQUIRE(plan && C && slice_max, RD_ERR_ARG);
  RD_REQUIRE(out_dtype == RD_F32 || out_dtype == RD_BF16, RD_ERR_DTYPE);
  const GemmPlan* p = static_cast<const GemmPlan*>(plan);
  RD_REQUIRE(p->N % 32 == 0 && slice_ld >= p->m_max, RD_ERR_SIZE);
  const int esz = out_dtype == RD_F32 ? 4 : 2;
  // the slice maxima are formed on the vector store path only
  RD_REQUIRE(((uintptr_t)C & 15) == 0 && (ldc * esz) % 16 == 0, RD_ERR_ALIGN);
  EpiArgs e{};
  e.C = C;
  e.ldc = ldc;
  e.part_val = slice_max;
  e.part_ld = slice_ld;
  return launch_epi(p, out_dtype, e, m_dev, kEpiSliceMax, status, (cudaStream_t)stream);
}

#ifdef RD_GEMM_TIMING
extern "C" __attribute__((visibility("default"))) int rd_gemm_set_timing(void* acc) {
  unsigned long long* p = static_cast<unsigned long long*>(acc);
  cudaError_t err = cudaMemcpyToSymbol(g_gemm_timing, &p, sizeof(p));
  RD_CHECK_CHAINED(err);
  return RD_OK;
}
#endif
