// FlashAttention forward on tcgen05 / TMEM with the score tile double-buffered, so that the
// tensor pipe computes S(j+1) = Q K(j+1)^T while the softmax of S(j) is still running.
//
// Same arithmetic as fa_tc.cu (the reference's loop nest, src/algorithms/flash_attention.cpp:277-450:
// tiles of S = Q K^T, online softmax with FP32 statistics, O += P V, key tiles above the causal
// diagonal skipped, :424), other schedule.  One CTA owns ONE 128-row query tile of one (batch, head):
//
//   TMEM (512 columns)   S[0] | S[1]  two score buffers, 128 fp32 columns each
//                        P[0] | P[1]  two probability buffers, 64 columns each (packed 16-bit pairs)
//                        O            head_dim fp32 columns
//   warps 0-3  softmax of the even key tiles (one thread per query row), P -> P[0]
//   warps 4-7  softmax of the odd key tiles, P -> P[1]
//   warp  8    lane 0 issues the tcgen05.mma of S = Q K^T, up to two key tiles ahead of the softmax
//   warp  9    lane 0 issues the tcgen05.mma of O += P V (two issuing threads: the waits and commits of
//              one overlap the MMAs of the other, so the tensor pipe is not idle while a thread waits)
//   warp 10    lane 0 issues the TMA loads (Q once, then K and V tiles through two rings)
//
// Because P has its own columns, a score buffer is free again as soon as its softmax warps have
// copied it to registers, and no softmax step waits for an MMA that depends on its own output: the
// chain softmax(j) -> PV(j) -> S(j+1) -> softmax(j+1) of the two-tile kernel is gone.
//
// Both softmax groups feed one accumulator, so all probabilities of a row use ONE reference maximum:
// the row maximum of key tile 0 (every query row sees key 0, so it is finite).  Using a reference
// below the true maximum is exact as long as 2^(growth) stays inside the range of the 16-bit format
// of P (the final division uses the row sum accumulated with the same reference).  A row whose scores
// later exceed the reference by more than the format's margin (a tile's partial row sum reaching 2^15
// for FP16, 2^64 for BF16) raises the CTA's entry in `redo`; the launcher always runs fa_tc.cu's kernel afterwards over the same grid
// of tiles, and that kernel recomputes exactly the flagged tiles with its rescaling softmax and
// returns at once for all others.
//
// Every wait is bounded, as in fa_tc.cu: a wait that gives up records a code in the device's error
// word, raises the CTA's abort flag, every role leaves its loop, TMEM is released, the kernel returns.
#include "fa_tc_common.cuh"

namespace ahpc {
namespace {

using namespace ptx;
using namespace tc;

constexpr int SOFTMAX_WARPS = 16;          // four groups of four warps
constexpr int TC2_THREADS = (SOFTMAX_WARPS + 4) * 32;   // + the three issuing warps and an idle one that completes their warpgroup
constexpr int S_WARP = SOFTMAX_WARPS, O_WARP = SOFTMAX_WARPS + 1, LOAD_WARP = SOFTMAX_WARPS + 2;
// The kernel is launched with 96 registers per thread (65536 / 640 rounded down to a multiple of 8); the issuing
// warpgroup then hands most of its share to the softmax warpgroups: 512 * 104 + 128 * 40 <= 640 * 96.
constexpr int SOFTMAX_REGS = 104, ISSUER_REGS = 40;
// Which of every 8 consecutive score pairs get their 2^x from poly_exp2_x2 (FMA pipe) instead of ex2 (special-
// function unit, 16 results per clock per SM - as many cycles per key tile as the two tensor-core contractions).
#ifndef AHPC_TC2_POLY
#define AHPC_TC2_POLY 0x0
#endif
#ifndef AHPC_TC2_PINGPONG
#define AHPC_TC2_PINGPONG 0
#endif
constexpr uint32_t POLY_PATTERN = AHPC_TC2_POLY;
constexpr bool EXP_TURNS = AHPC_TC2_PINGPONG != 0;

template <int D> struct Cfg2 {
    static constexpr int SUBTILES = D / 64;                  // 64-element (128-byte) wide column blocks
    static constexpr uint32_t TILE_BYTES = BN * D * 2;        // one Q, K or V tile
    static constexpr uint32_t SUB_BYTES = BN * 128;           // one 128-row x 128-byte swizzled block
    static constexpr int RING = D == 128 ? 3 : 6;             // depth of the K ring and of the V ring (tiles each)
    static constexpr int LEAD = 4;                            // S(i + LEAD) is issued right after O += P(i) V(i)
    static constexpr uint32_t SMEM_TILES = (1 + 2 * RING) * TILE_BYTES;
    static constexpr uint32_t AUX_BYTES = 3072;               // barriers + per-row exchange arrays
    static constexpr uint32_t SMEM_BYTES = SMEM_TILES + AUX_BYTES;   // 232448 for head_dim 128: all of an SM's shared memory
    static constexpr uint32_t P_COL = 256, O_COL = 384;
};

struct Tc2Params {
    void* out;
    float* lse;
    int batch, heads, seq_q, seq_kv;
    long long os[4];
    float scale, scale_log2;
    int causal;
    int n_tiles;
    int* error_word;
    int* redo;           // [tile][batch*heads]: 1 = recompute this tile with the rescaling kernel
#ifdef AHPC_TC2_PROF
    long long* prof;
    long long* trace;
    int trace_cta;
#endif
};

#ifdef AHPC_TC2_PROF
#define PROF_T0() const long long prof_t0_ = clock64()
#define PROF_ADD(slot) prof_acc[slot] += clock64() - prof_t0_
#define PROF_DECL() long long prof_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}
#define PROF_FLUSH(base) do { for (int q_ = 0; q_ < 8; ++q_) p.prof[(long long)blockIdx.x * 32 + (base) + q_] = prof_acc[q_]; } while (0)
#define TRACE(role, j, slot) do { if (blockIdx.x == p.trace_cta && (j) < 64) p.trace[((role) * 64 + (j)) * 8 + (slot)] = clock64(); } while (0)
#else
#define TRACE(role, j, slot)
#define PROF_T0()
#define PROF_ADD(slot)
#define PROF_DECL()
#define PROF_FLUSH(base)
#endif
#define WAITP(slot, ...) ([&] { PROF_T0(); const bool r_ = wait_bounded(__VA_ARGS__); PROF_ADD(slot); return r_; }())

struct Aux2 {            // lives behind the tiles in shared memory
    uint64_t q, s_full[2], s_free[2], p_full[2], p_free[2], o_done, m_ready, m_taken, l_ready, exp_done[2][4];
    uint64_t k_full[6], k_empty[6], v_full[6], v_empty[6];
    uint32_t tmem_base;
    int abort;
    int redo;
    // Row sums of the four softmax groups.  The first two rows of the array first carry the row maxima of key
    // tile 0 (left and right half of its columns); `m_taken` says that every group has read them.
    float l_part[4][BM];
};
static_assert(sizeof(Aux2) <= 3072, "Aux2 must fit its reserved bytes");

template <int D, bool BF16>
__global__ void __launch_bounds__(TC2_THREADS, 1)
fa_fwd_tc2_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                  const __grid_constant__ CUtensorMap map_v, const Tc2Params p) {
    using C = Cfg2<D>;
    // A tile's partial row sum at or above this means some probability left the range reserved for P
    // (FP16 holds up to 65504; BF16 shares the exponent range of FP32, 2^64 leaves room for the sums).
    constexpr float GROW_SUM_LIMIT = BF16 ? 1.8446744e19f : 32768.0f;
    extern __shared__ __align__(1024) uint8_t smem_raw[];     // 128-byte-swizzled tiles need 1024-byte alignment
    const uint32_t smem_base = smem_u32(smem_raw);
    uint8_t* smem_aligned = smem_raw;
    const uint32_t q_smem = smem_base;
    const uint32_t k_ring = smem_base + C::TILE_BYTES;
    const uint32_t v_ring = k_ring + C::RING * C::TILE_BYTES;
    Aux2* aux = reinterpret_cast<Aux2*>(smem_aligned + C::SMEM_TILES);
    volatile int* abort_flag = &aux->abort;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // Which (query tile, batch, head).  Consecutive CTAs are the query tiles of ONE (batch, head), so the CTAs
    // resident at any time share a few K/V streams and those stay in L2; heavy (late) tiles first when causal.
    const int bh_count = p.batch * p.heads;
    const int bh = blockIdx.x / p.n_tiles, tile_slot = blockIdx.x % p.n_tiles;
    const int tile = p.causal ? p.n_tiles - 1 - tile_slot : tile_slot;
    const int b = bh / p.heads, h = bh % p.heads;
    const int q0 = tile * BM;
    const int n_kv = kv_tiles_for(q0, p.seq_q, p.seq_kv, p.causal);

    if (threadIdx.x == S_WARP * 32) {
        mbar_init(smem_u32(&aux->q), 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&aux->s_full[i]), 1);
            mbar_init(smem_u32(&aux->s_free[i]), 8);
            mbar_init(smem_u32(&aux->p_full[i]), 8);
            mbar_init(smem_u32(&aux->p_free[i]), 1);
        }
        mbar_init(smem_u32(&aux->o_done), 1);
        mbar_init(smem_u32(&aux->m_ready), 8);
        mbar_init(smem_u32(&aux->m_taken), SOFTMAX_WARPS);
        mbar_init(smem_u32(&aux->l_ready), SOFTMAX_WARPS);
        for (int i = 0; i < 8; ++i) mbar_init(smem_u32(&aux->exp_done[i >> 2][i & 3]), 2);
        for (int s = 0; s < C::RING; ++s) {
            mbar_init(smem_u32(&aux->k_full[s]), 1);
            mbar_init(smem_u32(&aux->k_empty[s]), 1);
            mbar_init(smem_u32(&aux->v_full[s]), 1);
            mbar_init(smem_u32(&aux->v_empty[s]), 1);
        }
        aux->abort = (smem_base & 1023u) ? 1 : 0;              // misaligned tiles: every role leaves at its first wait
        if (aux->abort) atomicCAS(p.error_word, 0, 1001);
        aux->redo = 0;
        fence_mbar_init();
    }
    if (warp == S_WARP) {
        __syncwarp();
        tmem_alloc(smem_u32(&aux->tmem_base), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = aux->tmem_base;

    // The softmax threads hold a whole score row each; the issuing warpgroup gives them its spare registers.
    // (Each role's branch starts with its own setmaxnreg so that the register limit follows the role.)
    if (warp == LOAD_WARP) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(ISSUER_REGS));
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0 && n_kv > 0) {
            prefetch_tensormap(&map_q);
            prefetch_tensormap(&map_k);
            prefetch_tensormap(&map_v);
            {
                const uint32_t bar = smem_u32(&aux->q);
                mbar_expect_tx(bar, C::TILE_BYTES);
                for (int sub = 0; sub < C::SUBTILES; ++sub)
                    tma_load_4d(q_smem + sub * C::SUB_BYTES, &map_q, bar, sub * 64, q0, h, b);
            }
            // Loads follow the order in which the MMA warp consumes the tiles: K0..K3, then V(i), K(i+4).
            bool ok = true;
            PROF_DECL();
            const long long prof_start = clock64();
            int k_issued = 0, v_issued = 0;
            auto load_tile = [&](bool is_v, int j) {
                const int slot = j % C::RING, round = j / C::RING;
                uint64_t* full = is_v ? aux->v_full : aux->k_full;
                uint64_t* empty = is_v ? aux->v_empty : aux->k_empty;
                if (round > 0) ok = WAITP(is_v ? 1 : 0, smem_u32(&empty[slot]), (round - 1) & 1, abort_flag, p.error_word, (is_v ? 1110 : 1100) + slot);
                if (!ok) return;
                const uint32_t bar = smem_u32(&full[slot]);
#ifdef AHPC_TC2_EXP_SKIPLOAD
                if ((is_v && (AHPC_TC2_EXP_SKIPLOAD & 1)) || (!is_v && (AHPC_TC2_EXP_SKIPLOAD & 2))) {
                    if (j >= C::RING) { mbar_arrive(bar); if (is_v) v_issued = j + 1; else k_issued = j + 1; return; }
                }
#endif
                mbar_expect_tx(bar, C::TILE_BYTES);
                const uint32_t dst = (is_v ? v_ring : k_ring) + slot * C::TILE_BYTES;
                for (int sub = 0; sub < C::SUBTILES; ++sub)
                    tma_load_4d(dst + sub * C::SUB_BYTES, is_v ? &map_v : &map_k, bar, sub * 64, j * BN, h, b);
                if (is_v) v_issued = j + 1; else k_issued = j + 1;
                TRACE(0, j, is_v ? 1 : 0);
            };
            for (int j = 0; j < C::LEAD && j < n_kv && ok; ++j) load_tile(false, j);
            for (int i = 0; i < n_kv && ok; ++i) {
                load_tile(true, i);
                if (ok && i + C::LEAD < n_kv) load_tile(false, i + C::LEAD);
            }
#ifdef AHPC_TC2_PROF
            prof_acc[2] = clock64() - prof_start;
#endif
            PROF_FLUSH(0);
            if (!ok) {
                // Leave no copy in flight: wait (bounded) for the loads of the last ring round issued.
                for (int j = max(0, k_issued - C::RING); j < k_issued; ++j) {
                    long long t0 = clock64();
                    while (!mbar_try_wait(smem_u32(&aux->k_full[j % C::RING]), (j / C::RING) & 1) && clock64() - t0 < WAIT_LIMIT_CYCLES / 8) {}
                }
                for (int j = max(0, v_issued - C::RING); j < v_issued; ++j) {
                    long long t0 = clock64();
                    while (!mbar_try_wait(smem_u32(&aux->v_full[j % C::RING]), (j / C::RING) & 1) && clock64() - t0 < WAIT_LIMIT_CYCLES / 8) {}
                }
            }
        }
    } else if (warp == S_WARP) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(ISSUER_REGS));
        // ------------------------------------------------------------------ issuer of S = Q K^T
        if (lane == 0 && n_kv > 0) {
            constexpr uint32_t IDESC_S = idesc_f16(BF16 ? 1 : 0, BM, BN, 0, 0);     // Q (K-major) x K (K-major)
            bool ok = true;
            PROF_DECL();
            const long long prof_start = clock64();
            const uint64_t q_desc = smem_desc_sw128(q_smem, 16, 1024);
            ok = WAITP(0, smem_u32(&aux->q), 0, abort_flag, p.error_word, 1200);
            // S[j & 1] = Q K_j^T : head_dim/16 MMAs of K = 16.  Needs K_j in shared memory and, from j = 2 on,
            // the softmax warps of tile j-2 to have copied that buffer out.
            for (int j = 0; j < n_kv && ok; ++j) {
                const int slot = j % C::RING, buf = j & 1;
                TRACE(1, j, 0);
                ok = WAITP(1, smem_u32(&aux->k_full[slot]), (j / C::RING) & 1, abort_flag, p.error_word, 1220);
                if (ok && j >= 2) ok = WAITP(2, smem_u32(&aux->s_free[buf]), ((j - 2) >> 1) & 1, abort_flag, p.error_word, 1230 + buf);
                if (!ok) break;
                tc_fence_after_sync();
                const uint64_t k_desc = smem_desc_sw128(k_ring + slot * C::TILE_BYTES, 16, 1024);
                TRACE(1, j, 1);
                { PROF_T0();
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint64_t off = ((kk >> 2) * C::SUB_BYTES + (kk & 3) * 32) >> 4;   // descriptor addresses count 16 bytes
                    mma_ss(tmem + buf * BN, q_desc + off, k_desc + off, IDESC_S, kk > 0);
                }
                PROF_ADD(6); }
                tc_commit(smem_u32(&aux->s_full[buf]));
                tc_commit(smem_u32(&aux->k_empty[slot]));
                TRACE(1, j, 2);
            }
#ifdef AHPC_TC2_PROF
            prof_acc[5] = clock64() - prof_start;
#endif
            PROF_FLUSH(8);
        }
    } else if (warp == O_WARP) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(ISSUER_REGS));
        // ------------------------------------------------------------------ issuer of O += P V
        if (lane == 0 && n_kv > 0) {
            constexpr uint32_t IDESC_O = idesc_f16(BF16 ? 1 : 0, BM, D, 0, 1);      // P (TMEM) x V (MN-major)
            bool ok = true;
            PROF_DECL();
            const long long prof_start = clock64();
            // O (+)= P[j & 1] V_j : 8 MMAs of K = 16 keys; V is MN-major (head_dim contiguous)
            for (int j = 0; j < n_kv && ok; ++j) {
                const int slot = j % C::RING, buf = j & 1;
                TRACE(2, j, 0);
                ok = WAITP(3, smem_u32(&aux->v_full[slot]), (j / C::RING) & 1, abort_flag, p.error_word, 1240);
                if (ok) ok = WAITP(4, smem_u32(&aux->p_full[buf]), (j >> 1) & 1, abort_flag, p.error_word, 1250 + buf);
                if (!ok) break;
                tc_fence_after_sync();
                const uint64_t v_desc = smem_desc_sw128(v_ring + slot * C::TILE_BYTES, C::SUB_BYTES, 1024);
                TRACE(2, j, 1);
                { PROF_T0();
#pragma unroll
                for (int kk = 0; kk < BN / 16; ++kk)
                    mma_ts(tmem + C::O_COL, tmem + C::P_COL + buf * 64 + kk * 8, v_desc + (uint64_t)((kk * 16 * 128) >> 4), IDESC_O,
                           !(j == 0 && kk == 0));
                PROF_ADD(7); }
                tc_commit(smem_u32(&aux->p_free[buf]));
                tc_commit(smem_u32(&aux->v_empty[slot]));
                TRACE(2, j, 2);
            }
            if (ok) tc_commit(smem_u32(&aux->o_done));
#ifdef AHPC_TC2_PROF
            prof_acc[5] = clock64() - prof_start;
#endif
            PROF_FLUSH(24);
        }
    } else if (warp > LOAD_WARP) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(ISSUER_REGS));
    } else {
        // ------------------------------------------------------------------ softmax + epilogue
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(SOFTMAX_REGS));
        // Four groups of four warps.  Group wg works on the key tiles of parity g = wg & 1 and, of each such tile,
        // on the 64 columns of half hc = wg >> 1; warp w of every group owns the TMEM lanes (query rows) 32 w .. 32 w + 31,
        // one thread per row.  So each scheduler (4 warps sharing the same rows) always has two warps in their
        // exponentials while the other two wait, load or store.
        const int wg = warp >> 2, g = wg & 1, hc = wg >> 1, quad = warp & 3;
        const int r_in_tile = quad * 32 + lane;
        const int row = q0 + r_in_tile;
        const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
        const uint32_t s_addr = tmem + lane_base + g * BN + hc * 64;
        const uint32_t p_addr = tmem + lane_base + C::P_COL + g * 64 + hc * 32;
        const uint32_t o_addr = tmem + lane_base + C::O_COL;
        float m_ref = 0.f, l_run = 0.f;
        bool ok = true, grew = false, took_m = false;
        PROF_DECL();
        const long long prof_start = clock64();

        int i = 0;
        const bool tracer = quad == 0 && hc == 0 && lane == 0;
        (void)tracer;
        const uint64_t scale2 = pack_f2(p.scale_log2, p.scale_log2);
        for (int j = g; j < n_kv; j += 2, ++i) {
            if (tracer) TRACE(3 + g, j, 0);
            ok = WAITP(0, smem_u32(&aux->s_full[g]), i & 1, abort_flag, p.error_word, 1300 + g);
            if (!ok) break;
            tc_fence_after_sync();
            if (tracer) TRACE(3 + g, j, 1);

            const int k0 = j * BN + hc * 64;                                            // first key of this warp's columns
            const bool need_mask = (p.causal && j * BN + BN - 1 > q0) || (j * BN + BN > p.seq_kv);
            const int limit = p.causal ? min(p.seq_kv - 1, row) : p.seq_kv - 1;         // last visible key
            uint32_t sr[2][32];
            tmem_ld32(s_addr, sr[0]);
            tmem_ld32(s_addr + 32, sr[1]);
            tmem_wait_ld();
            // this warp's copy of its part of S[g] is complete: the buffer may take the tile after next
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&aux->s_free[g]));
            if (tracer) TRACE(3 + g, j, 2);
            if (need_mask) {
#pragma unroll
                for (int c = 0; c < 2; ++c)
#pragma unroll
                    for (int e = 0; e < 32; ++e)
                        if (k0 + c * 32 + e > limit) sr[c][e] = 0xff800000u;            // -inf
            }
            if (j == 0) {
                // Key tile 0 fixes the reference maximum of the row for all groups: the two halves meet in shared memory.
                float mx[2];
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    mx[c] = -INFINITY;
#pragma unroll
                    for (int e = 0; e < 32; e += 2) mx[c] = max3(mx[c], __uint_as_float(sr[c][e]), __uint_as_float(sr[c][e + 1]));
                }
                aux->l_part[hc][r_in_tile] = fmaxf(mx[0], mx[1]);
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&aux->m_ready));
            }
            if (i == 0) {
                ok = WAITP(2, smem_u32(&aux->m_ready), 0, abort_flag, p.error_word, 1320);
                if (!ok) break;
                m_ref = fmaxf(aux->l_part[0][r_in_tile], aux->l_part[1][r_in_tile]);
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&aux->m_taken));
                took_m = true;
            }
            if (i >= 1) {          // P[g] may still feed the PV MMA of this parity's previous tile (normally long done)
                ok = WAITP(1, smem_u32(&aux->p_free[g]), (i - 1) & 1, abort_flag, p.error_word, 1330 + g);
                if (!ok) break;
                tc_fence_after_sync();
            }
            uint64_t negm2 = pack_f2(-m_ref * p.scale_log2, -m_ref * p.scale_log2);
            if (EXP_TURNS && j >= 1) {
                // The exponentials of consecutive key tiles take turns on each scheduler's special-function unit.
                ok = WAITP(5, smem_u32(&aux->exp_done[g ^ 1][quad]), ((j - 1) >> 1) & 1, abort_flag, p.error_word, 1360 + g);
                if (!ok) break;
                asm volatile("" : "+l"(negm2));          // the exponentials below stay behind the wait
            }
            if (tracer) TRACE(3 + g, j, 3);
            uint64_t sum2[4] = {0ull, 0ull, 0ull, 0ull};                                // four packed partial row sums
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                // In three passes (arguments, exponentials, sums and packing), so that the warp issues a run of
                // independent ex2 before the first instruction that needs one of their results.
                uint64_t x2[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) x2[e] = fma2(pack_u2(sr[c][2 * e], sr[c][2 * e + 1]), scale2, negm2);
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    if ((POLY_PATTERN >> (e & 7)) & 1u) {
                        x2[e] = poly_exp2_x2(x2[e]);
                    } else {
                        x2[e] = pack_f2(fast_exp2(__uint_as_float((uint32_t)x2[e])), fast_exp2(__uint_as_float((uint32_t)(x2[e] >> 32))));
                    }
                }
                uint32_t packed[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    sum2[e & 3] = add2(sum2[e & 3], x2[e]);
                    packed[e] = pack2<BF16>(__uint_as_float((uint32_t)x2[e]), __uint_as_float((uint32_t)(x2[e] >> 32)));
                }
                tmem_st16(p_addr + c * 16, packed);
            }
            const uint64_t tot = add2(add2(sum2[0], sum2[1]), add2(sum2[2], sum2[3]));
            const float psum = __uint_as_float((uint32_t)tot) + __uint_as_float((uint32_t)(tot >> 32));
            // the arrival takes the row sum as an operand, which keeps it behind the last exponential
            if (EXP_TURNS && lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&aux->exp_done[g][quad])), "f"(psum) : "memory");
            if (tracer) TRACE(3 + g, j, 4);
            // A probability beyond the range reserved for P means the reference maximum is too stale for this row.
            grew |= !(psum < GROW_SUM_LIMIT);
            l_run += psum;
            tmem_wait_st();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&aux->p_full[g]));
            if (tracer) TRACE(3 + g, j, 6);
        }
        if (grew) aux->redo = 1;
#ifdef AHPC_TC2_PROF
        prof_acc[3] = clock64() - prof_start;
#endif

        // The row sums of the four groups meet in shared memory, in the array that carried the maxima of key tile 0:
        // first make sure every group has taken those.
        if (!took_m) {
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&aux->m_taken));
        }
        if (ok) ok = WAITP(4, smem_u32(&aux->m_taken), 0, abort_flag, p.error_word, 1335);
        if (ok) aux->l_part[wg][r_in_tile] = l_run;
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&aux->l_ready));
        if (ok) ok = WAITP(4, smem_u32(&aux->l_ready), 0, abort_flag, p.error_word, 1340);
        if (ok) ok = WAITP(4, smem_u32(&aux->o_done), 0, abort_flag, p.error_word, 1350);
        if (ok) {
            // each group stores a quarter of the columns of O
            tc_fence_after_sync();
            const float l_tot = (aux->l_part[0][r_in_tile] + aux->l_part[1][r_in_tile]) + (aux->l_part[2][r_in_tile] + aux->l_part[3][r_in_tile]);
            const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
            constexpr int QUART = D / 4;
            uint16_t* orow_g = static_cast<uint16_t*>(p.out) + b * p.os[0] + h * p.os[1] + (long long)row * p.os[2] + wg * QUART;
            uint32_t orow[QUART];
            if constexpr (QUART == 32) tmem_ld32(o_addr + wg * QUART, orow);      // warp-collective: rows past seq_q still take part
            else tmem_ld16(o_addr + wg * QUART, orow);
            tmem_wait_ld();
            if (row < p.seq_q) {
#pragma unroll
                for (int e = 0; e < QUART / 8; ++e) {
                    uint4 v;
                    v.x = pack2<BF16>(__uint_as_float(orow[8 * e + 0]) * inv, __uint_as_float(orow[8 * e + 1]) * inv);
                    v.y = pack2<BF16>(__uint_as_float(orow[8 * e + 2]) * inv, __uint_as_float(orow[8 * e + 3]) * inv);
                    v.z = pack2<BF16>(__uint_as_float(orow[8 * e + 4]) * inv, __uint_as_float(orow[8 * e + 5]) * inv);
                    v.w = pack2<BF16>(__uint_as_float(orow[8 * e + 6]) * inv, __uint_as_float(orow[8 * e + 7]) * inv);
                    *reinterpret_cast<uint4*>(orow_g + e * 8) = v;
                }
            }
            if (wg == 0 && p.lse && row < p.seq_q)
                p.lse[((long long)b * p.heads + h) * p.seq_q + row] = l_tot > 0.f ? m_ref * p.scale + logf(l_tot) : -INFINITY;
        }
#ifdef AHPC_TC2_PROF
        prof_acc[5] = clock64() - prof_start;
        if (warp == 0 && lane == 0) PROF_FLUSH(16);
#endif
    }

    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0) p.redo[(long long)tile * bh_count + bh] = (aux->redo || aux->abort) ? 1 : 0;
    if (warp == S_WARP) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

#ifdef AHPC_TC2_PROF
long long* g_prof = nullptr;
long long g_prof_ctas = 0;
long long* tc2_prof_buffer(long long ctas) {
    if (ctas > g_prof_ctas) {
        if (g_prof) cudaFree(g_prof);
        cudaMalloc(&g_prof, ctas * 32 * sizeof(long long));
        g_prof_ctas = ctas;
    }
    cudaMemset(g_prof, 0, ctas * 32 * sizeof(long long));
    return g_prof;
}
long long* g_trace = nullptr;
int g_trace_cta = 0;
#endif

template <int D, bool BF16>
ahpc_status launch2(const FaLaunch& a, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const Tc2Params& p) {
    using C = Cfg2<D>;
    auto kernel = fa_fwd_tc2_kernel<D, BF16>;
    AHPC_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM_BYTES));
    const long long ctas = (long long)p.n_tiles * a.batch * a.heads;
    kernel<<<(unsigned)ctas, TC2_THREADS, C::SMEM_BYTES, a.stream>>>(mq, mk, mv, p);
    AHPC_CUDA_OK(cudaGetLastError());
    return AHPC_SUCCESS;
}

}  // namespace

ahpc_status launch_fa_tc2(const FaLaunch& a, int* redo_flags) {
    CUtensorMap mq, mk, mv;
    AHPC_TRY(make_map(&mq, a.q, a.dtype, a.batch, a.heads, a.seq_q, a.head_dim, a.qs));
    AHPC_TRY(make_map(&mk, a.k, a.dtype, a.batch, a.heads, a.seq_kv, a.head_dim, a.ks));
    AHPC_TRY(make_map(&mv, a.v, a.dtype, a.batch, a.heads, a.seq_kv, a.head_dim, a.vs));
    Tc2Params p;
    p.out = a.out; p.lse = a.lse;
    p.batch = a.batch; p.heads = a.heads; p.seq_q = a.seq_q; p.seq_kv = a.seq_kv;
    for (int i = 0; i < 4; ++i) p.os[i] = a.os[i];
    p.scale = a.scale;
    p.scale_log2 = a.scale * 1.4426950408889634f;
    p.causal = a.causal;
    p.n_tiles = (a.seq_q + BM - 1) / BM;
    p.redo = redo_flags;
#ifdef AHPC_TC2_PROF
    p.prof = tc2_prof_buffer((long long)p.n_tiles * a.batch * a.heads);
    if (!g_trace) cudaMalloc(&g_trace, 5 * 64 * 8 * sizeof(long long));
    cudaMemset(g_trace, 0, 5 * 64 * 8 * sizeof(long long));
    p.trace = g_trace;
    p.trace_cta = g_trace_cta;
#endif
    AHPC_TRY(error_word_for(a.device, &p.error_word));
    const bool bf16 = a.dtype == AHPC_BF16;
    if (a.head_dim == 128) return bf16 ? launch2<128, true>(a, mq, mk, mv, p) : launch2<128, false>(a, mq, mk, mv, p);
    return bf16 ? launch2<64, true>(a, mq, mk, mv, p) : launch2<64, false>(a, mq, mk, mv, p);
}

}  // namespace ahpc

#ifdef AHPC_TC2_PROF
// experiment builds only: copies the per-CTA cycle counters of the last launch to the host
extern "C" __attribute__((visibility("default"))) long long ahpc_tc2_prof_read(long long* out, long long max_ctas) {
    using namespace ahpc;
    cudaDeviceSynchronize();
    const long long n = g_prof_ctas < max_ctas ? g_prof_ctas : max_ctas;
    cudaMemcpy(out, g_prof, n * 32 * sizeof(long long), cudaMemcpyDeviceToHost);
    return n;
}
extern "C" __attribute__((visibility("default"))) void ahpc_tc2_trace_read(long long* out, int next_cta) {
    using namespace ahpc;
    cudaDeviceSynchronize();
    if (g_trace) cudaMemcpy(out, g_trace, 5 * 64 * 8 * sizeof(long long), cudaMemcpyDeviceToHost);
    g_trace_cta = next_cta;
}
#endif
