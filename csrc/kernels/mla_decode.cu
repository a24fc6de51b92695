// MLA absorbed-weight decode attention over a paged latent cache (tcgen05 + TMEM, sm_100a).
//
//   q      [Bq, H, 576]  bf16   absorbed query: 512 latent dims | 64 rope dims
//   cache  [slots, 576]  bf16   one "KV head": normalised latent c_kv (512) | roped k_pe (64); keys are
//                               the full 576-wide row, values are its first 512 entries
//   out    [Bq, H, 512]  bf16   softmax(q k^T * scale) v   (still in latent space; W_UV follows)
//
// Work split.  The q heads of one row are the UMMA M dimension (128 lanes, one head per TMEM lane and
// per softmax thread, so row max / row sum never leave the thread).  The fp32 output accumulator of 128
// heads x 512 dims would fill all of TMEM, so two CTAs (blockIdx.x = 0/1) each own 256 output dims;
// both compute the full score tile.  blockIdx.y splits the KV range (flash-decoding), blockIdx.z = q row.
//
// Per CTA: warp 0 = TMA producer, warps 1 and 10 = MMA issuers (even / odd tiles), warps 2..9 = softmax /
// correction / epilogue.
//   S = Q K^T     A = Q  (smem, K-major, 9 chunks of 64 dims)   B = KV tile (smem, K-major)      -> TMEM
//   P = softmax   written back to TMEM as packed bf16 (A operand of the second MMA)
//   O += P V      A = P  (TMEM)                                  B = KV tile (same smem, MN-major) -> TMEM
// KV tiles are 64 tokens, two of them in flight: the score MMA of tile i+1 runs on the tensor pipe while the
// softmax warps work on tile i (two S buffers in TMEM), and P V of tile i follows as soon as P is written.
// Five of the nine 64-dim q chunks sit in shared memory, the other four in TMEM (as A operands), which
// leaves 144 KB for KV staging.  Each 64-dim chunk of a tile has its own full/empty barrier pair: the chunks
// that only the score MMA reads (the other CTA's value dims and the rope dims) go through a small ring and
// are refilled as soon as S is issued, the value chunks sit in one of three stages until P V has run.
// The running max is only raised when it grows by more than 2^8 (lazy rescale), so the O accumulator is
// rarely read back.
//
// Stands where the reference calls npu_fused_infer_attention_score on the absorbed path
// (omni/models/common/layers/attention/deepseek_mla.py:533-560, 625-650).
#include "../include/omni_noalloc.h"
#include "../include/omni_ptx.cuh"
#include "../include/tma_host.h"

namespace omni {

struct MlaDecodeParams {
  int H;
  int block_size;
  const int* block_table;
  int bt_ld;
  const int* seq_lens;   // [Bq] visible kv tokens of each q row
  const int* q_to_seq;   // [Bq] block-table row of each q row, or null (identity)
  const __nv_bfloat16* q; // [Bq, H, 576] (also read directly for the chunks kept in TMEM)
  float scale_log2;      // softmax scale * log2(e)
  int num_splits;
  __nv_bfloat16* out;    // [Bq, H, 512]
  float* o_part;         // [Bq, splits, H, 512]
  float* lse_part;       // [Bq, splits, H]   (log2 domain)
  OmniStatus* status;
};

constexpr int MLA_TILE = 64;                          // kv tokens per tile
constexpr int MLA_CHUNK_BYTES = MLA_TILE * 128;       // 64 tokens x 64 dims bf16 = 8 KB
// KV staging, 144 KB: this CTA's four value chunks of a tile are needed until its P V has run, the other five
// chunks only until the score MMA has read them.  The value chunks cycle through three 32 KB stages, the
// score-only chunks through a ring of six 8 KB slots, so every load is issued about one tile ahead of its use.
constexpr int MLA_VSTAGES = 3;
constexpr int MLA_VSTAGE_BYTES = 4 * MLA_CHUNK_BYTES;
constexpr int MLA_NSLOTS = 6;
constexpr int MLA_KV_BYTES = MLA_VSTAGES * MLA_VSTAGE_BYTES + MLA_NSLOTS * MLA_CHUNK_BYTES;
constexpr int MLA_Q_CHUNK = 128 * 128;                // 128 heads x 64 dims bf16
constexpr int MLA_QS = 5;   // q chunks in shared memory: this CTA's four value-dim chunks and the rope chunk;
// the other half's four latent chunks are kept in TMEM (packed bf16), two written by each softmax group
constexpr int MLA_SMEM =
    MLA_QS * MLA_Q_CHUNK + MLA_KV_BYTES + 1536 /*barriers + softmax exchange*/ + 1024 /*align*/;
static_assert(MLA_SMEM <= 232448, "exceeds the 227 KB shared-memory limit of one CTA");
// warp 0 TMA, warps 1 and 10 MMA issue (even and odd tiles), warps 2..9 softmax (two groups of four, 32 score columns each)
constexpr int MLA_THREADS = 352;
// TMEM columns: O accumulator | two S tiles (P, packed bf16, overwrites half of each group's own S columns) |
// four packed-bf16 q chunks
constexpr int TM_O = 0, TM_S = 256, TM_Q = 384, TM_COLS = 512;

enum { MS_Q = 31, MS_KV_EMPTY, MS_KV_FULL, MS_P_FULL, MS_S_FULL, MS_O_DONE, MS_QT, MS_TMEM, MS_SC_ISSUED };

__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}


// What every warp was waiting for when a CTA gave up: the first CTA of a process whose wait runs out leaves this
// record (read and cleared by omni_mla_debug_read), so that a time-out can be told from its report alone.
//   [0] taken  [1..3] blockIdx x, y, z  [4] tiles of the CTA  [5] kv_len  [6] first tile  [7] num_splits
//   [8 + w] warp w: (site << 16) | detail of the wait it left, 0 if it was not waiting
__device__ int g_mla_debug[32];
constexpr int MLA_DBG_INTS_AFTER_ABORT = 27;   // the per-warp words sit at byte 320 of the barrier block

__device__ __forceinline__ bool mla_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, OmniStatus* st, int site,
                                         int detail) {
  const bool ok = mbar_wait(bar, parity, abort_flag, st, site, detail);
  if (!ok) const_cast<int*>(abort_flag)[MLA_DBG_INTS_AFTER_ABORT + (threadIdx.x >> 5)] = (site << 16) | (detail & 0xffff);
  return ok;
}

// ---------------------------------------------------------------------------------------------------------
// Producer and MMA roles.  Both walk the same sequence of KV chunks with a few running counters (no division,
// no tables), and their loops are kept small: a tcgen05.mma issues in about 50 cycles from a short loop whose
// descriptors are a uniform base plus a small offset, but far slower from long unrolled code.
//
// KV chunk c = latent dims 64c..64c+63 (c < 8) or the rope dims (c = 8).  CTA half h owns the value chunks
// 4h..4h+3 and accumulates those 256 output dims.  Per tile, in this order:
//   1. the four latent chunks of the other half (score MMA only; their q chunks sit in TMEM),
//   2. the rope chunk (score MMA only; q chunk in shared memory slot 4),
//   3. this half's four value chunks (q chunks in shared memory slots 0..3), which stay in their stage until
//      P V of the tile has run.
// Chunks of kinds 1 and 2 go through a ring of MLA_NSLOTS 8 KB slots, kind 3 through MLA_VSTAGES stages.
// ---------------------------------------------------------------------------------------------------------
struct MlaPipe {
  uint32_t sq_addr, kv_addr;
  uint64_t *kv_full, *kv_empty, *s_full, *p_full, *o_done, *o_final, *sc_issued;
  volatile int* abort_flag;
  OmniStatus* status;
};
struct MlaRing {   // position in the score-only ring / the value stages
  uint32_t slot = 0, par = 0, vstage = 0, vpar = 0;
  __device__ __forceinline__ void next_slot() { if (++slot == MLA_NSLOTS) { slot = 0; par ^= 1u; } }
  __device__ __forceinline__ void next_stage() { if (++vstage == MLA_VSTAGES) { vstage = 0; vpar ^= 1u; } }
  __device__ __forceinline__ void skip_tile() {   // a tile that another issuer walks through
    slot += 5;
    if (slot >= MLA_NSLOTS) { slot -= MLA_NSLOTS; par ^= 1u; }
    next_stage();
  }
};

template <int HALF>
__device__ __forceinline__ void mla_producer(const MlaPipe& px, const CUtensorMap* tmap_kv, const int* bt, int block_size,
                                             int box_rows, int kv_len, int tile_begin, int n) {
  MlaRing rg;
#pragma unroll 1
  for (int i = 0; i < n; ++i) {
    const int tok0 = (tile_begin + i) * MLA_TILE;
    // cache rows of this tile's TMA boxes (pages past the end of the sequence repeat the last valid page;
    // their scores are masked)
    int rows[MLA_TILE / 32];
#pragma unroll
    for (int r = 0; r < MLA_TILE / 32; ++r) {
      const int tok = tok0 + r * 32;
      const int pg = min(tok, kv_len - 1) / block_size;
      rows[r] = bt[pg] * block_size + tok % block_size;
    }
#pragma unroll 1
    for (int oc = 0; oc < 5; ++oc) {
      const int c = oc < 4 ? (1 - HALF) * 4 + oc : 8;
      uint64_t* full = &px.kv_full[MLA_VSTAGES + rg.slot];
      if (!mla_wait(&px.kv_empty[MLA_VSTAGES + rg.slot], rg.par ^ 1u, px.abort_flag, px.status, MS_KV_EMPTY, (i << 8) | c)) return;
      mbar_expect_tx(full, MLA_CHUNK_BYTES);
      const uint32_t dst = px.kv_addr + MLA_VSTAGES * MLA_VSTAGE_BYTES + rg.slot * MLA_CHUNK_BYTES;
      if (box_rows == MLA_TILE) tma_load_2d_addr(dst, tmap_kv, full, c * 64, rows[0]);
      else {
#pragma unroll
        for (int r = 0; r < MLA_TILE / 32; ++r) tma_load_2d_addr(dst + r * 32 * 128, tmap_kv, full, c * 64, rows[r]);
      }
      rg.next_slot();
    }
    {
      uint64_t* full = &px.kv_full[rg.vstage];
      if (!mla_wait(&px.kv_empty[rg.vstage], rg.vpar ^ 1u, px.abort_flag, px.status, MS_KV_EMPTY, (i << 8) | (100 + (int)rg.vstage))) return;
      mbar_expect_tx(full, MLA_VSTAGE_BYTES);
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        const uint32_t dst = px.kv_addr + rg.vstage * MLA_VSTAGE_BYTES + v * MLA_CHUNK_BYTES;
        if (box_rows == MLA_TILE) tma_load_2d_addr(dst, tmap_kv, full, (HALF * 4 + v) * 64, rows[0]);
        else {
#pragma unroll
          for (int r = 0; r < MLA_TILE / 32; ++r)
            tma_load_2d_addr(dst + r * 32 * 128, tmap_kv, full, (HALF * 4 + v) * 64, rows[r]);
        }
      }
      rg.next_stage();
    }
  }
}

// S = Q K^T of the next tile in the score stream, into S buffer `buf`.  Run by the whole MMA warp; one
// elected lane issues.
__device__ __forceinline__ bool mla_issue_scores(const MlaPipe& px, MlaRing& rg, const uint32_t buf, const int tile) {
  constexpr uint32_t idesc_qk = umma_idesc(128, MLA_TILE, 1, 1, 0, 0);
  const uint32_t d_s = TM_S + buf * 64;
  const uint64_t qdesc0 = umma_desc_kmajor_sw128(px.sq_addr);
  const uint64_t ring0 = umma_desc_kmajor_sw128(px.kv_addr + MLA_VSTAGES * MLA_VSTAGE_BYTES);
  const uint64_t vdesc0 = umma_desc_kmajor_sw128(px.kv_addr);
#pragma unroll 1
  for (int oc = 0; oc < 5; ++oc) {
    if (!mla_wait(&px.kv_full[MLA_VSTAGES + rg.slot], rg.par, px.abort_flag, px.status, MS_KV_FULL, (tile << 8) | oc)) return false;
    tc_fence_after();
    const uint64_t bd = ring0 + (uint64_t)(rg.slot * (MLA_CHUNK_BYTES >> 4));
    if (elect_one()) {
      if (oc < 4) {
        const uint32_t at = TM_Q + oc * 32;
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_bf16_ts(d_s, at + 8 * k, bd + 2 * k, idesc_qk, (oc > 0 || k > 0) ? 1u : 0u);
      } else {
        const uint64_t ad = qdesc0 + (uint64_t)((4 * MLA_Q_CHUNK) >> 4);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_bf16(d_s, ad + 2 * k, bd + 2 * k, idesc_qk, 1u);
      }
      umma_commit(&px.kv_empty[MLA_VSTAGES + rg.slot]);   // the slot can be refilled
    }
    __syncwarp();
    rg.next_slot();
  }
  if (!mla_wait(&px.kv_full[rg.vstage], rg.vpar, px.abort_flag, px.status, MS_KV_FULL, (tile << 8) | (100 + (int)rg.vstage))) return false;
  tc_fence_after();
  if (elect_one()) {
    const uint64_t vd = vdesc0 + (uint64_t)(rg.vstage * (MLA_VSTAGE_BYTES >> 4));
#pragma unroll
    for (int v = 0; v < 4; ++v) {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        umma_bf16(d_s, qdesc0 + (uint64_t)(v * (MLA_Q_CHUNK >> 4) + 2 * k), vd + (uint64_t)(v * (MLA_CHUNK_BYTES >> 4) + 2 * k),
                  idesc_qk, 1u);
    }
    umma_commit(&px.s_full[buf]);
    mbar_arrive(&px.sc_issued[buf]);   // every chunk of this tile has landed: the other issuer may look at the ring again
  }
  __syncwarp();
  rg.next_stage();
  return true;
}

// MMA issue for the tiles i = which, which + 2, ...  Issuing a score tile costs one lane about 1700 cycles (36
// instructions of about 48), as much as the tensor pipe needs to execute a whole tile, so two warps share the work:
// while one waits for the softmax of its tile and issues P V, the other issues the scores of the next tile.
// Tile i uses S buffer i & 1, so each issuer always works on the same buffer.
__device__ __forceinline__ void mla_mma(const MlaPipe& px, int n, const int which) {
  constexpr uint32_t idesc_pv = umma_idesc(128, 256, 1, 1, 0, 1);
  MlaRing rg;
  if (which) rg.skip_tile();
  uint32_t pv_stage = (uint32_t)which;       // i % MLA_VSTAGES
  const uint32_t buf = (uint32_t)which;
  const uint64_t vdesc0 = umma_desc_mnmajor_sw128(px.kv_addr, MLA_CHUNK_BYTES, 1024);
#pragma unroll 1
  for (int i = which; i < n; i += 2) {
    // A ring slot (and a value stage) is filled for the two issuers in turn, and a parity wait can only tell the
    // current fill from the one before it.  The fill before "mine" belongs to the previous tile, which the other
    // issuer consumes; if it has not landed yet when this warp arrives (TMA loads complete in any order), the wait for
    // mine would see the fill two back as "complete" and pass on stale data, and the releases that follow wedge the
    // ring.  So this warp first waits until the other one has seen every chunk of the previous tile land.
    if (i >= 1 && !mla_wait(&px.sc_issued[buf ^ 1u], ((uint32_t)(i - 1) >> 1) & 1u, px.abort_flag, px.status, MS_SC_ISSUED, i)) return;
    if (!mla_issue_scores(px, rg, buf, i)) return;
    rg.skip_tile();
    // the first P V zero-initialises the accumulator: the other issuer's first P V must enter the pipe after it
    if (i == 1 && !mla_wait(px.o_done, 0u, px.abort_flag, px.status, MS_O_DONE, 0)) return;
    // ---- O += P V
    if (!mla_wait(&px.p_full[buf], ((uint32_t)i >> 1) & 1u, px.abort_flag, px.status, MS_P_FULL, i)) return;
    tc_fence_after();
    if (elect_one()) {
      // 16 tokens per MMA: two 8-token groups of 1024 B; dims advance by whole 8 KB chunks.  P of tokens
      // 0..31 sits in columns 0..15 of the S buffer, P of tokens 32..63 in columns 32..47.
      const uint64_t vd = vdesc0 + (uint64_t)(pv_stage * (MLA_VSTAGE_BYTES >> 4));
      const uint32_t pbase = TM_S + buf * 64;
      umma_bf16_ts(TM_O, pbase, vd, idesc_pv, i > 0 ? 1u : 0u);
#pragma unroll
      for (int k = 1; k < MLA_TILE / 16; ++k)
        umma_bf16_ts(TM_O, pbase + (k >> 1) * 32 + (k & 1) * 8, vd + (uint64_t)(k * 128), idesc_pv, 1u);
      umma_commit(&px.kv_empty[pv_stage]);
      umma_commit(px.o_done);
      if (i + 2 >= n) umma_commit(px.o_final);   // this issuer's last tile
    }
    __syncwarp();
    pv_stage += 2;
    if (pv_stage >= MLA_VSTAGES) pv_stage -= MLA_VSTAGES;
  }
}

__global__ void __launch_bounds__(MLA_THREADS, 1)
mla_decode_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_kv,
                  const MlaDecodeParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sq = smem;
  uint8_t* skv = smem + MLA_QS * MLA_Q_CHUNK;
  uint64_t* bars = (uint64_t*)(skv + MLA_KV_BYTES);
  uint64_t* q_full = bars;                          // 1
  uint64_t* kv_full = bars + 1;                     // [3 value stages] then [6 score-only slots]
  uint64_t* kv_empty = kv_full + 9;                 // same layout
  uint64_t* s_full = kv_empty + 9;                  // 2, one per S buffer
  uint64_t* p_full = s_full + 2;                    // 2
  uint64_t* o_done = p_full + 2;                    // 1
  uint64_t* o_final = o_done + 1;                   // 1: all P V of this CTA retired (one arrival per issuer)
  uint64_t* qt_full = o_final + 1;                  // 1: q chunks written to TMEM
  uint64_t* sc_issued = bars + 30;                  // 2, one per issuer: the scores of its current tile are all issued
  uint32_t* tmem_slot = (uint32_t*)(qt_full + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  int* sm_counter = (int*)(tmem_slot + 2);          // softmax group rendezvous (only grows)
  __nv_bfloat16* sm_max = (__nv_bfloat16*)(bars + 64);  // [2 tile parities][2 groups][128 rows] row maxima, 1 KB
  float* sm_sum = (float*)(bars + 64);                  // [2 groups][128 rows], same 1 KB after the last tile

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int half = blockIdx.x;   // which 256 output dims
  const int split = blockIdx.y;
  const int bq = blockIdx.z;

  const int kv_len = p.seq_lens[bq];
  const int tiles_total = (kv_len + MLA_TILE - 1) / MLA_TILE;
  const int tps = (tiles_total + p.num_splits - 1) / p.num_splits;
  const int tile_begin = split * tps;
  const int tile_end = min(tiles_total, tile_begin + tps);
  const int n = max(0, tile_end - tile_begin);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int c = 0; c < 9; ++c) {
      mbar_init(&kv_full[c], 1);
      mbar_init(&kv_empty[c], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&p_full[b], 8);
    }
    mbar_init(&sc_issued[0], 1);
    mbar_init(&sc_issued[1], 1);
    mbar_init(o_done, 1);
    mbar_init(o_final, n >= 2 ? 2 : 1);   // the last P V of each issuer that has tiles
    mbar_init(qt_full, 8);
    *abort_flag = 0;
    *sm_counter = 0;
    for (int w = 0; w < 12; ++w) const_cast<int*>(abort_flag)[MLA_DBG_INTS_AFTER_ABORT + w] = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // the whole TMEM (512 columns) is allocated, so the base can only be column 0 of lane 0; keeping it a
  // literal keeps every TMEM address of the MMA role a compile-time constant
  constexpr uint32_t tmem_base = 0;
  if (*tmem_slot != 0u) {
    if (threadIdx.x == 0) { *abort_flag = 1; report_status(p.status, OMNI_ERR_MBAR_TIMEOUT, MS_TMEM, (int)*tmem_slot); }
    __syncthreads();
    if (warp == 1) tmem_dealloc(*tmem_slot, TM_COLS);
    return;
  }

  const int box_rows = min(p.block_size, MLA_TILE);   // tokens per TMA box (one cache page, at most a tile)

  if (n > 0) {
    if (warp == 0) {
      if (lane == 0) {
        const MlaPipe px{smem_u32(sq), smem_u32(skv), kv_full, kv_empty, s_full, p_full, o_done, o_final, sc_issued, abort_flag, p.status};
        tma_prefetch_desc(&tmap_q);
        tma_prefetch_desc(&tmap_kv);
        // q chunks in shared memory: this half's four value-dim chunks (slots 0..3) and the rope chunk (slot 4)
        mbar_expect_tx(q_full, MLA_QS * MLA_Q_CHUNK);
        for (int c = 0; c < 4; ++c) tma_load_2d(sq + c * MLA_Q_CHUNK, &tmap_q, q_full, (half * 4 + c) * 64, bq * p.H);
        tma_load_2d(sq + 4 * MLA_Q_CHUNK, &tmap_q, q_full, 512, bq * p.H);
        const int seq = p.q_to_seq ? p.q_to_seq[bq] : bq;
        const int* bt = p.block_table + (size_t)seq * p.bt_ld;
        if (half == 0) mla_producer<0>(px, &tmap_kv, bt, p.block_size, box_rows, kv_len, tile_begin, n);
        else mla_producer<1>(px, &tmap_kv, bt, p.block_size, box_rows, kv_len, tile_begin, n);
      }
    } else if (warp == 1 || warp == 10) {
      const MlaPipe px{smem_u32(sq), smem_u32(skv), kv_full, kv_empty, s_full, p_full, o_done, o_final, sc_issued, abort_flag, p.status};
      bool ok = mla_wait(q_full, 0, abort_flag, p.status, MS_Q, 0);
      if (ok) ok = mla_wait(qt_full, 0, abort_flag, p.status, MS_QT, 0);
      tc_fence_after();
      if (ok) mla_mma(px, n, warp == 1 ? 0 : 1);
    } else {
      // ------------------------------------------------------------ softmax / correction / epilogue
      // Eight warps: lane quadrant qd = warp & 3 selects 32 heads, group grp selects 32 of the 64 score
      // columns (and 128 of the 256 output columns).  The two warps that share a quadrant exchange their
      // row maxima through shared memory once per tile; row sums are only combined at the very end.
      const int qd = warp & 3;
      const int grp = (warp - 2) >> 2;
      const int row = qd * 32 + lane;  // head
      const uint32_t lane_addr = tmem_base + ((uint32_t)(qd * 32) << 16);
      float m = -INFINITY, l = 0.f;
      bool ok = true;
      int sync_no = 0;
      // rendezvous of all eight softmax warps; watches the abort flag so that nobody can be stranded
      auto group_sync = [&]() -> bool {
        __syncwarp();
        if (lane == 0) { __threadfence_block(); atomicAdd(sm_counter, 1); }
        ++sync_no;
        uint32_t spins = 0;
        while (*(volatile int*)sm_counter < 8 * sync_no) {
          if (((++spins) & 0xff) == 0 && *abort_flag) {
            const_cast<int*>(abort_flag)[MLA_DBG_INTS_AFTER_ABORT + warp] = (99 << 16) | (sync_no & 0xffff);
            return false;
          }
        }
        __syncwarp();
        return true;
      };
      // this head's q values for the chunks kept in TMEM (the other half's 256 latent dims), as packed bf16
      // pairs; group g writes two of the four chunks
      {
        const uint4* qsrc = reinterpret_cast<const uint4*>(p.q + ((size_t)bq * p.H + row) * 576 + (1 - half) * 256);
        const bool row_ok = row < p.H;
#pragma unroll 1
        for (int c = grp * 2; c < grp * 2 + 2; ++c) {
          uint32_t v[32];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint4 x = row_ok ? __ldg(qsrc + c * 8 + j) : make_uint4(0, 0, 0, 0);
            v[4 * j] = x.x; v[4 * j + 1] = x.y; v[4 * j + 2] = x.z; v[4 * j + 3] = x.w;
          }
          tmem_st_x32(lane_addr + TM_Q + c * 32, v);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(qt_full);
      }
      for (int i = 0; i < n; ++i) {
        const int st = i & 1;
        if (!mla_wait(&s_full[st], (i >> 1) & 1, abort_flag, p.status, MS_S_FULL, i)) { ok = false; break; }
        tc_fence_after();
        const int valid = kv_len - (tile_begin + i) * MLA_TILE - grp * 32;  // valid columns of this group's half
        const uint32_t s_addr = lane_addr + TM_S + st * 64 + grp * 32;
        float s[32];
        {
          uint32_t sv[32];
          tmem_ld_x32(s_addr, sv);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) s[j] = (j < valid) ? __uint_as_float(sv[j]) * p.scale_log2 : -INFINITY;
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          mx4[0] = fmaxf(mx4[0], s[j]); mx4[1] = fmaxf(mx4[1], s[j + 1]);
          mx4[2] = fmaxf(mx4[2], s[j + 2]); mx4[3] = fmaxf(mx4[3], s[j + 3]);
        }
        const float mx_local = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        // the slab alternates with the tile parity: a warp may already write tile i+1's maxima while its
        // partner still reads tile i's (one rendezvous per tile separates the writes of tiles i and i+2).
        // Both warps of a row read both (bf16-rounded) entries, so they agree on the reference exactly; the
        // reference only has to be near the true maximum, not equal to it.
        __nv_bfloat16* slab = sm_max + st * 256;
        slab[grp * 128 + row] = __float2bfloat16_rn(mx_local);
        if (!group_sync()) { ok = false; break; }
        const float mx = fmaxf(__bfloat162float(slab[row]), __bfloat162float(slab[128 + row]));
        const float m_new = fmaxf(m, mx);
        const bool grow = (m_new - m) > 8.0f;  // also true on the first tile (m = -inf)
        if (i == 0) {
          m = m_new;
        } else if (__any_sync(0xffffffffu, grow)) {
          // P V of the previous tile must have retired before O is touched; P V of this tile waits for P
          if (!mla_wait(o_done, (i - 1) & 1, abort_flag, p.status, MS_O_DONE, i)) { ok = false; break; }
          tc_fence_after();
          const float f = grow ? exp2f(m - m_new) : 1.0f;
          if (grow) { l *= f; m = m_new; }
#pragma unroll 1
          for (int c = grp * 128; c < grp * 128 + 128; c += 32) {
            uint32_t ov[32];
            tmem_ld_x32(lane_addr + TM_O + c, ov);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) ov[j] = __float_as_uint(__uint_as_float(ov[j]) * f);
            tmem_st_x32(lane_addr + TM_O + c, ov);
          }
          tmem_st_wait();
        }
        float rs4[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          float p0, p1;
          const float a0 = s[2 * j] - m, a1 = s[2 * j + 1] - m;
          asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p0) : "f"(a0));
          asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p1) : "f"(a1));
          rs4[j & 3] += p0 + p1;
          __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
          pk[j] = *reinterpret_cast<uint32_t*>(&h2);
        }
        l += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
        // P (packed bf16) overwrites the first half of this group's own S columns, which only its warps read
        tmem_st_x16(s_addr, pk);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[st]);
      }
      // o_done flips once per tile and is only sampled when a rescale is needed, so its parity cannot
      // tell "last tile retired" from "two tiles behind"; the single-use o_final barrier can.
      if (ok) ok = mla_wait(o_final, 0, abort_flag, p.status, MS_O_DONE, n);
      if (ok) ok = group_sync();   // every warp is past its last read of the maxima slabs
      if (ok) {
        sm_sum[grp * 128 + row] = l;
        ok = group_sync();
      }
      if (ok) {
        tc_fence_after();
        const float inv_l = 1.0f / (sm_sum[row] + sm_sum[128 + row]);
        const float l_tot = sm_sum[row] + sm_sum[128 + row];
        const bool row_ok = row < p.H;
        const int c_lo = grp * 128;
        if (p.num_splits == 1) {
          __nv_bfloat16* orow = p.out + ((size_t)bq * p.H + row) * 512 + half * 256;
#pragma unroll 1
          for (int c = c_lo; c < c_lo + 128; c += 32) {
            uint32_t ov[32];
            tmem_ld_x32(lane_addr + TM_O + c, ov);
            tmem_ld_wait();
            if (row_ok) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                __nv_bfloat16 o8[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) o8[e] = __float2bfloat16(__uint_as_float(ov[j + e]) * inv_l);
                *reinterpret_cast<uint4*>(orow + c + j) = *reinterpret_cast<uint4*>(o8);
              }
            }
          }
        } else {
          float* orow = p.o_part + (((size_t)bq * p.num_splits + split) * p.H + row) * 512 + half * 256;
#pragma unroll 1
          for (int c = c_lo; c < c_lo + 128; c += 32) {
            uint32_t ov[32];
            tmem_ld_x32(lane_addr + TM_O + c, ov);
            tmem_ld_wait();
            if (row_ok) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                float4 o4 = make_float4(__uint_as_float(ov[j]) * inv_l, __uint_as_float(ov[j + 1]) * inv_l,
                                        __uint_as_float(ov[j + 2]) * inv_l, __uint_as_float(ov[j + 3]) * inv_l);
                *reinterpret_cast<float4*>(orow + c + j) = o4;
              }
            }
          }
          if (half == 0 && grp == 0 && row_ok)
            p.lse_part[((size_t)bq * p.num_splits + split) * p.H + row] = m + log2f(l_tot);
        }
      }
    }
  } else if (warp >= 2 && warp < 6) {
    // empty KV range for this split (or an empty / padding row): neutral partial result
    const int row = (warp & 3) * 32 + lane;
    if (row < p.H) {
      if (p.num_splits == 1) {
        __nv_bfloat16* orow = p.out + ((size_t)bq * p.H + row) * 512 + half * 256;
        for (int c = 0; c < 256; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0, 0, 0, 0);
      } else {
        float* orow = p.o_part + (((size_t)bq * p.num_splits + split) * p.H + row) * 512 + half * 256;
        for (int c = 0; c < 256; c += 4) *reinterpret_cast<float4*>(orow + c) = make_float4(0.f, 0.f, 0.f, 0.f);
        if (half == 0) p.lse_part[((size_t)bq * p.num_splits + split) * p.H + row] = -INFINITY;
      }
    }
  }

  if (*abort_flag) {
    if (threadIdx.x == 0) report_abort(abort_flag, p.status);
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0 && atomicCAS(&g_mla_debug[0], 0, 1) == 0) {
    g_mla_debug[1] = blockIdx.x; g_mla_debug[2] = blockIdx.y; g_mla_debug[3] = blockIdx.z;
    g_mla_debug[4] = n; g_mla_debug[5] = kv_len; g_mla_debug[6] = tile_begin; g_mla_debug[7] = p.num_splits;
    for (int w = 0; w < 12; ++w) g_mla_debug[8 + w] = const_cast<int*>(abort_flag)[MLA_DBG_INTS_AFTER_ABORT + w];
    // bit b set = "the phase of parity 0 of barrier b has completed" (i.e. the barrier now runs an odd phase)
    int full_odd = 0, empty_odd = 0, misc = 0;
    for (int c = 0; c < 9; ++c) {
      full_odd |= (int)mbar_try_wait(&kv_full[c], 0) << c;
      empty_odd |= (int)mbar_try_wait(&kv_empty[c], 0) << c;
    }
    misc |= (int)mbar_try_wait(&s_full[0], 0) | ((int)mbar_try_wait(&s_full[1], 0) << 1) | ((int)mbar_try_wait(&p_full[0], 0) << 2) |
            ((int)mbar_try_wait(&p_full[1], 0) << 3) | ((int)mbar_try_wait(o_done, 0) << 4) | ((int)mbar_try_wait(o_final, 0) << 5);
    g_mla_debug[20] = full_odd; g_mla_debug[21] = empty_odd; g_mla_debug[22] = misc;
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TM_COLS);
  }
}

// out[bq, h, :] = sum_s w_s * o_part[bq, s, h, :],  w_s = 2^(lse_s - max) / sum
__global__ void mla_combine_kernel(const float* __restrict__ o_part, const float* __restrict__ lse_part,
                                   int splits, int H, __nv_bfloat16* out) {
  const int bh = blockIdx.x;  // bq * H + h
  const int bq = bh / H, h = bh - bq * H;
  float mx = -INFINITY;
  for (int s = 0; s < splits; ++s) mx = fmaxf(mx, lse_part[((size_t)bq * splits + s) * H + h]);
  float den = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float v = lse_part[((size_t)bq * splits + s) * H + h];
    den += (v == -INFINITY) ? 0.f : exp2f(v - mx);
  }
  const float inv = den > 0.f ? 1.f / den : 0.f;
  for (int c = threadIdx.x * 4; c < 512; c += blockDim.x * 4) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < splits; ++s) {
      const float v = lse_part[((size_t)bq * splits + s) * H + h];
      if (v == -INFINITY) continue;
      const float w = exp2f(v - mx) * inv;
      const float4 o = *reinterpret_cast<const float4*>(o_part + (((size_t)bq * splits + s) * H + h) * 512 + c);
      acc.x += w * o.x; acc.y += w * o.y; acc.z += w * o.z; acc.w += w * o.w;
    }
    __nv_bfloat16 o4[4] = {__float2bfloat16(acc.x), __float2bfloat16(acc.y), __float2bfloat16(acc.z),
                           __float2bfloat16(acc.w)};
    *reinterpret_cast<uint2*>(out + (size_t)bh * 512 + c) = *reinterpret_cast<uint2*>(o4);
  }
}

}  // namespace omni

using namespace omni;


// Copies the record of the first CTA whose wait ran out (32 ints, all zero if none did) and clears it.
extern "C" int omni_mla_debug_read(int* out32) {
  cudaError_t e = cudaMemcpyFromSymbol(out32, g_mla_debug, sizeof(int) * 32);
  if (e != cudaSuccess) return (int)e;
  static const int zeros[32] = {0};
  return (int)cudaMemcpyToSymbol(g_mla_debug, zeros, sizeof(zeros));
}

// Scratch needed for num_splits > 1: o_part = Bq*splits*H*512 floats, lse_part = Bq*splits*H floats.
extern "C" int omni_mla_decode(const void* q, const void* cache, int cache_ld, long long num_slots,
                               const int* block_table, int bt_ld, const int* seq_lens, const int* q_to_seq, int Bq,
                               int H, int block_size, float scale, int num_splits, void* out, float* o_part,
                               float* lse_part, void* status, cudaStream_t stream) {
  if (Bq <= 0) return 0;
  if (H < 1 || H > 128) return -1;
  if (block_size != 32 && block_size % 64 != 0) return -2;
  if (num_splits < 1) return -3;
  if (num_splits > 1 && (o_part == nullptr || lse_part == nullptr)) return -4;
  CUtensorMap tq, tkv;
  if (make_tmap_2d(&tq, q, 2, (uint64_t)Bq * H, 576, 576, 128, 64, true)) return -10;
  const int box_rows = block_size < MLA_TILE ? block_size : MLA_TILE;
  if (make_tmap_2d(&tkv, cache, 2, (uint64_t)num_slots, 576, cache_ld, box_rows, 64, true)) return -11;
  MlaDecodeParams p;
  p.q = (const __nv_bfloat16*)q; p.H = H; p.block_size = block_size; p.block_table = block_table; p.bt_ld = bt_ld; p.seq_lens = seq_lens;
  p.q_to_seq = q_to_seq; p.scale_log2 = scale * 1.4426950408889634f; p.num_splits = num_splits;
  p.out = (__nv_bfloat16*)out; p.o_part = o_part; p.lse_part = lse_part; p.status = (OmniStatus*)status;
  static bool configured[64] = {false};
  if (int e = ensure_dyn_smem((const void*)mla_decode_kernel, MLA_SMEM, configured)) return e;
  dim3 grid(2, num_splits, Bq);
  mla_decode_kernel<<<grid, MLA_THREADS, MLA_SMEM, stream>>>(tq, tkv, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  if (num_splits > 1) {
    mla_combine_kernel<<<Bq * H, 128, 0, stream>>>(o_part, lse_part, num_splits, H, (__nv_bfloat16*)out);
    e = cudaGetLastError();
  }
  return (int)e;
}

// -------------------------------------------------------------------------------------------------------
// Allocation-free variant (see omni_noalloc.h): the split-KV scratch is a fixed array inside the library.
// In host code the array's name is only a stand-in for the symbol, not a device address; the address each
// GPU gave it is fetched once per device with cudaGetSymbolAddress and passed to the kernels.
// -------------------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_mla_noalloc_scratch[OMNI_MLA_NOALLOC_SCRATCH_BYTES];

static unsigned char* noalloc_scratch_for_current_device(int* rc) {
  static unsigned char* per_device[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) { *rc = e != cudaSuccess ? (int)e : -101; return nullptr; }
  if (per_device[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_mla_noalloc_scratch);   // set-up: once per device, with that device current
    if (e != cudaSuccess || p == nullptr) { *rc = e != cudaSuccess ? (int)e : -102; return nullptr; }
    per_device[dev] = (unsigned char*)p;
  }
  *rc = 0;
  return per_device[dev];
}

extern "C" int omni_mla_decode_noalloc(const void* q, const void* cache, int cache_ld, long long num_slots,
                                       const int* block_table, int bt_ld, const int* seq_lens, const int* q_to_seq,
                                       int Bq, int H, int block_size, float scale, int num_splits, void* out,
                                       void* status, cudaStream_t stream) {
  if (Bq <= 0) return 0;
  if (num_splits < 1 || H < 1) return -3;
  const unsigned long long parts = (unsigned long long)Bq * (unsigned long long)num_splits * (unsigned long long)H;
  // one split writes `out` directly and never touches the scratch, so the limit only binds split-KV calls
  if (num_splits > 1 && (parts * 512ull * 4ull > (unsigned long long)OMNI_MLA_NOALLOC_OPART_BYTES ||
                         parts > (unsigned long long)OMNI_MLA_NOALLOC_LSE_FLOATS)) {
    fprintf(stderr,
            "omni_mla_decode_noalloc: Bq*num_splits*H = %llu exceeds the built-in scratch (limit %u); "
            "use omni_mla_decode with caller-provided scratch\n",
            parts, (unsigned)(OMNI_MLA_NOALLOC_OPART_BYTES / (512u * 4u)));
    return OMNI_NOALLOC_TOO_LARGE;
  }
  int rc = 0;
  unsigned char* scratch = noalloc_scratch_for_current_device(&rc);
  if (scratch == nullptr) return rc;
  float* o_part = reinterpret_cast<float*>(scratch);
  float* lse_part = reinterpret_cast<float*>(scratch + OMNI_MLA_NOALLOC_OPART_BYTES);
  // num_splits == 1 writes `out` directly and leaves the scratch untouched; the pointers are passed either way
  return omni_mla_decode(q, cache, cache_ld, num_slots, block_table, bt_ld, seq_lens, q_to_seq, Bq, H, block_size,
                         scale, num_splits, out, o_part, lse_part, status, stream);
}
