// Grouped-query decode on the tensor cores with the KEYS along the rows of the MMA tile.
//
// One query token per sequence; the G query heads that share a key/value head (G <= 16) attend to that head's keys
// together, so K and V cross HBM once per group (paged_attention_kernel of the reference reads them once per query
// head, src/backends/cuda/cuda_kernels.cu:416-514).  Per 128-key tile:
//     S^T[128 keys x 16 heads] = K[128 x D] . Q^T[D x 16]        A = the page blocks as the pool keeps them, B = Q
//     softmax along the keys: a thread owns one key (one tensor-memory lane) and the 16 heads' scores of it
//     O^T[D x 16 heads]       += V^T[D x 128 keys] . P^T[128 x 16]  A = the value tile (head_dim contiguous), B = P^T
// so every lane that computes an exponential computes one that is used - the form with the heads along the rows
// (MODE_DECODE of fa_fwd_tc_kernel) spends 128-row MMAs and 128-column softmax rows on G useful rows.
//
// A CTA takes items (chunk of a context, key/value head, sequence) w = blockIdx.x, blockIdx.x + gridDim.x, ... as one stream
// of key tiles; the library launches one CTA per item.  Measured (64 sequences of 512..8192 tokens, 8 key/value heads):
// 4.5 TB/s for any group size up to 16, the same as the heads-along-the-rows form - about 4 us per CTA plus 1.7 us per tile
// and SM - where the FP32 kernels, whose loads land in the registers of many small CTAs, stream at 6.3 TB/s for one head
// per key/value head.  Neither the MMA nor the softmax work bounds it (this form has almost none); deeper rings, page ids
// fetched per chunk instead of per tile, one persistent CTA per SM, and asking the pages of later tiles into L2 ahead of the
// ring (cp.async.bulk.prefetch.L2: 20 % slower) did not help.
// 320 threads: warps 0-3 and 4-7 are two softmax groups that take an item's key
// tiles alternately, each with its own running maximum / sum per head and its own accumulator O^T; warp 8 issues the MMAs,
// warp 9 the copies (one bulk copy per page of keys, one TMA box per page and 128-byte column block of values).  Each group
// leaves one partial (maximum, sum, O) per query head for paged_combine_kernel.  head_dim 128, page size 16, FP16 / BF16.
//
// Every wait is bounded (fa_tc_common.cuh: wait_bounded): a barrier that does not complete records a code in the device's
// error word, raises the CTA's abort flag, and every role leaves its loop; tensor memory is released before the CTA ends.
#include <algorithm>

#include "fa_tc_common.cuh"

namespace ahpc {
namespace {

using namespace ptx;
using namespace tc;

constexpr int D = 128;                       // head_dim
constexpr int HP = 16;                       // heads per tile (the group, padded)
constexpr int KV_STAGES = 3;
constexpr uint32_t TILE_BYTES = BN * D * 2;  // one K or V tile
constexpr uint32_t Q_BYTES = HP * D * 2;     // 16 heads x 256 bytes, as two 128-byte-swizzled column blocks of 2 KB; two buffers
constexpr uint32_t PT_BYTES = HP * BN * 2;   // P^T of one group: 16 heads x 128 keys
constexpr uint32_t SMEM_Q = 0, SMEM_PT = SMEM_Q + 2 * Q_BYTES, SMEM_K = 16384, SMEM_V = SMEM_K + KV_STAGES * TILE_BYTES;
constexpr uint32_t SMEM_BARS = SMEM_V + KV_STAGES * TILE_BYTES;
constexpr uint32_t SMEM_TOTAL = SMEM_BARS + 1024 /*barriers, exchange*/ + 1024 /*alignment slack*/;
constexpr uint32_t TMEM_DECODE_COLS = 64;    // S^T of the two groups at columns 0 / 16, O^T at 32 / 48

struct Bars {
    uint64_t q_full[2], q_empty[2], k_full[KV_STAGES], k_empty[KV_STAGES], v_full[KV_STAGES], v_empty[KV_STAGES], s_full[2], p_full[2], o_done[2];
    uint64_t exchanged[2];                   // per group: its four warps have put their values into `red`
    uint32_t tmem_base;
    int abort;
    float red[2][4][HP];                     // per group and warp: the tile's maximum per head; later the sums
};

struct DecodeTcParams {
    const uint16_t* k_data;
    const int32_t* table;
    const int32_t* seq_ids;
    const int32_t* seq_len;
    float* part_o;            // [n_seqs][parts][q_heads][D]
    float2* part_ml;          // [n_seqs][parts][q_heads]
    long long page_elems;
    int max_pages, q_heads, kv_heads, n_seqs, group, split, chunks, parts, n_items;
    float scale_log2;
    int* error_word;
};

// One unit of work: a chunk of one sequence's context for one key/value head.  Every role of the CTA walks the same list
// (item w, w + gridDim.x, ...) and skips the chunks that lie past the sequence's end.
struct Item {
    int si, kvh, chunk, kv_base, seq_kv, n_kv, n_pages, page_base;
    const int32_t* table_row;
    bool valid;
};
__device__ __forceinline__ Item get_item(const DecodeTcParams& p, int w) {
    Item it;
    // chunk fastest (measured: 10 % faster with one CTA per item than sequence-fastest, which is what a CTA that walks
    // several items would want - with gridDim.x a multiple of the chunk count it would otherwise see one chunk index only)
    it.chunk = w % p.chunks;
    const int r = w / p.chunks;
    it.kvh = r % p.kv_heads;
    it.si = r / p.kv_heads;
    const int seq = __ldg(p.seq_ids + it.si);
    const int len = __ldg(p.seq_len + seq);
    it.kv_base = it.chunk * p.split;
    it.valid = it.kv_base < len;
    it.seq_kv = min(len, it.kv_base + p.split);          // keys [kv_base, seq_kv) are this item's
    it.n_kv = (it.seq_kv - it.kv_base + BN - 1) / BN;
    it.n_pages = (it.seq_kv + 15) >> 4;
    it.page_base = it.kv_base >> 4;
    it.table_row = p.table + (long long)seq * p.max_pages;
    return it;
}

__device__ __forceinline__ int ordered(float x) {
    const int i = __float_as_int(x);
    return i >= 0 ? i : i ^ 0x7fffffff;
}
__device__ __forceinline__ float unordered(int i) { return __int_as_float(i >= 0 ? i : i ^ 0x7fffffff); }

template <bool BF16>
__global__ void __launch_bounds__(TC_THREADS, 1)
paged_decode_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_v, const DecodeTcParams p) {
    if (gridDim.x == (unsigned)p.n_items && !get_item(p, blockIdx.x).valid) return;      // one item per CTA, and it lies past the sequence's end
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
    Bars* bars = reinterpret_cast<Bars*>(smem + SMEM_BARS);
    volatile int* abort_flag = &bars->abort;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = p.group;

    if (threadIdx.x == MMA_WARP * 32) {
        bars->abort = 0;
        for (int s = 0; s < KV_STAGES; ++s) {
            mbar_init(smem_u32(&bars->k_full[s]), 1); mbar_init(smem_u32(&bars->k_empty[s]), 1);
            mbar_init(smem_u32(&bars->v_full[s]), 1); mbar_init(smem_u32(&bars->v_empty[s]), 1);
        }
        for (int g = 0; g < 2; ++g) {
            mbar_init(smem_u32(&bars->q_full[g]), 1);
            mbar_init(smem_u32(&bars->q_empty[g]), 1);
            mbar_init(smem_u32(&bars->s_full[g]), 1);
            mbar_init(smem_u32(&bars->p_full[g]), BM);
            mbar_init(smem_u32(&bars->o_done[g]), 1);
            mbar_init(smem_u32(&bars->exchanged[g]), 4);
        }
        fence_mbar_init();
    }
    if (warp == MMA_WARP) {
        __syncwarp();
        tmem_alloc(smem_u32(&bars->tmem_base), TMEM_DECODE_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = bars->tmem_base;

    if (warp == TMA_WARP) {
        // ------------------------------------------------------------------ copies: runs ahead of the other roles, across items
        if (lane == 0) {
            prefetch_tensormap(&map_q);
            prefetch_tensormap(&map_v);
        }
        bool ok = true;
        int tiles = 0, items = 0, issued_k = 0, issued_v = 0;      // running counts over the CTA's items
        for (int w = blockIdx.x; w < p.n_items && ok; w += gridDim.x) {
            const Item it = get_item(p, w);
            if (!it.valid) continue;
            const int qb = items & 1;
            if (items >= 2) ok = wait_bounded(smem_u32(&bars->q_empty[qb]), ((items >> 1) - 1) & 1, abort_flag, p.error_word, 520 + qb);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (lane == 0) {
                const uint32_t bar = smem_u32(&bars->q_full[qb]);
                mbar_expect_tx(bar, Q_BYTES);
                const int row0 = it.si * p.q_heads + it.kvh * G;          // the group's first head in the [n_seqs * q_heads, D] view of q
                for (int sub = 0; sub < 2; ++sub) tma_load_4d(smem_base + SMEM_Q + qb * Q_BYTES + sub * (HP * 128), &map_q, bar, sub * 64, row0, 0, 0);
            }
            for (int j = 0; j < it.n_kv; ++j, ++tiles) {
                const int st = tiles % KV_STAGES, round = tiles / KV_STAGES;
                const int first = it.page_base + j * (BN / 16), valid = min(BN / 16, it.n_pages - first);
                if (round > 0) ok = wait_bounded(smem_u32(&bars->k_empty[st]), (round - 1) & 1, abort_flag, p.error_word, 500 + st);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                int page = 0;
                if (lane == 0) mbar_expect_tx(smem_u32(&bars->k_full[st]), valid * (16 * D * 2));
                if (lane < valid) {
                    page = __ldg(it.table_row + first + lane);
                    bulk_load(smem_base + SMEM_K + st * TILE_BYTES + lane * (16 * D * 2),
                              p.k_data + (long long)page * p.page_elems + (long long)it.kvh * 16 * D, 16 * D * 2, smem_u32(&bars->k_full[st]));
                }
                issued_k = tiles + 1;
                if (round > 0) ok = wait_bounded(smem_u32(&bars->v_empty[st]), (round - 1) & 1, abort_flag, p.error_word, 510 + st);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (lane == 0) mbar_expect_tx(smem_u32(&bars->v_full[st]), valid * (16 * D * 2));
                if (lane < valid)
                    for (int sub = 0; sub < 2; ++sub)
                        tma_load_4d(smem_base + SMEM_V + st * TILE_BYTES + sub * (BN * 128) + lane * 16 * 128, &map_v, smem_u32(&bars->v_full[st]),
                                    sub * 64, 0, it.kvh, page);
                issued_v = tiles + 1;
            }
            ++items;
        }
        if (!ok && lane == 0) {
            // leave no copy in flight: wait (bounded) for what the last ring round asked for
            for (int t = max(0, issued_k - KV_STAGES); t < issued_k; ++t) {
                long long t0 = clock64();
                while (!mbar_try_wait(smem_u32(&bars->k_full[t % KV_STAGES]), (t / KV_STAGES) & 1) && clock64() - t0 < WAIT_LIMIT_CYCLES / 8) {}
            }
            for (int t = max(0, issued_v - KV_STAGES); t < issued_v; ++t) {
                long long t0 = clock64();
                while (!mbar_try_wait(smem_u32(&bars->v_full[t % KV_STAGES]), (t / KV_STAGES) & 1) && clock64() - t0 < WAIT_LIMIT_CYCLES / 8) {}
            }
        }
    } else if (warp == MMA_WARP) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t IDESC_S = idesc_f16(BF16 ? 1 : 0, BM, HP, 0, 0);     // K (K-major, unswizzled) x Q (K-major)
            constexpr uint32_t IDESC_O = idesc_f16(BF16 ? 1 : 0, BM, HP, 1, 0);     // V^T (head_dim contiguous) x P^T (K-major, unswizzled)
            bool ok = true;
            int done[2] = {0, 0};                                        // key tiles group g has been given P V for
            // S^T_g = K_j Q^T : 8 steps of 16 elements of the head dimension
            auto issue_s = [&](int g, int st, int qb) {
                const uint32_t ka = smem_base + SMEM_K + st * TILE_BYTES, qa = smem_base + SMEM_Q + qb * Q_BYTES;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk)
                    mma_ss(tmem + g * HP, smem_desc_plain(ka + kk * 256, 128, D * 16),
                           smem_desc_sw128(qa + (kk >> 2) * (HP * 128) + (kk & 3) * 32, 16, 1024), IDESC_S, kk > 0);
                tc_commit(smem_u32(&bars->s_full[g]));
                tc_commit(smem_u32(&bars->k_empty[st]));
            };
            // O^T_g (+)= V_j^T P^T_g : one step per page (16 keys) the tile holds
            auto issue_o = [&](int g, int st, bool first, int steps) {
                const uint32_t va = smem_base + SMEM_V + st * TILE_BYTES, pa = smem_base + SMEM_PT + g * PT_BYTES;
#pragma unroll
                for (int kk = 0; kk < BN / 16; ++kk)
                    if (kk < steps)
                        mma_ss(tmem + 2 * HP + g * HP, smem_desc_sw128(va + kk * 16 * 128, BN * 128, 1024),
                               smem_desc_plain(pa + kk * 256, 128, BN * 16), IDESC_O, !(first && kk == 0));
                tc_commit(smem_u32(&bars->o_done[g]));
                tc_commit(smem_u32(&bars->v_empty[st]));
            };
            // The CTA's key tiles form one stream across its items; tile t of the stream belongs to group t & 1.  Order on the
            // pipe: S(0) S(1) | PV(0) S(2) | PV(1) S(3) | ... - the S of the next item's first tiles go out before the last
            // P V of this one, so the softmax groups never wait for an item to drain.
            struct Cursor { int w, j, items; Item it; bool end; };
            auto next_item = [&](Cursor& c) {
                c.j = 0;
                for (c.w += gridDim.x; c.w < p.n_items; c.w += gridDim.x) {
                    c.it = get_item(p, c.w);
                    if (c.it.valid) return;
                }
                c.end = true;
            };
            Cursor a{(int)blockIdx.x - (int)gridDim.x, 0, 0, Item{}, false};
            next_item(a);
            Cursor b = a;                                                // b runs two tiles ahead of a and issues the S
            int ta = 0, tb = 0;                                          // stream positions of a and b
            auto s_step = [&]() {
                if (b.end || !ok) return;
                const int qb = b.items & 1;
                if (b.j == 0) ok = wait_bounded(smem_u32(&bars->q_full[qb]), (b.items >> 1) & 1, abort_flag, p.error_word, 600 + qb);
                if (ok) ok = wait_bounded(smem_u32(&bars->k_full[tb % KV_STAGES]), (tb / KV_STAGES) & 1, abort_flag, p.error_word, 610);
                if (!ok) return;
                tc_fence_after_sync();
                issue_s(tb & 1, tb % KV_STAGES, qb);
                ++tb;
                if (++b.j == b.it.n_kv) {
                    tc_commit(smem_u32(&bars->q_empty[qb]));             // every S of the item has been issued: Q may go when they are through
                    ++b.items;
                    next_item(b);
                }
            };
            s_step();
            s_step();
            while (!a.end && ok) {
                const int g = ta & 1, st = ta % KV_STAGES;
                ok = wait_bounded(smem_u32(&bars->v_full[st]), (ta / KV_STAGES) & 1, abort_flag, p.error_word, 620);
                if (ok) ok = wait_bounded(smem_u32(&bars->p_full[g]), done[g] & 1, abort_flag, p.error_word, 630 + g);
                if (!ok) break;
                tc_fence_after_sync();
                issue_o(g, st, a.j < 2, min(BN / 16, a.it.n_pages - a.it.page_base - a.j * (BN / 16)));
                ++done[g];
                ++ta;
                if (++a.j == a.it.n_kv) next_item(a);
                s_step();
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax along the keys + the item's partial
        const int g = warp >> 2, wq = warp & 3;                 // group; warp quadrant of tensor memory
        const int key_in_tile = wq * 32 + lane;                 // this thread's key (S^T) and, later, its element of the head dimension (O^T)
        const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
        const uint32_t s_addr = tmem + lane_base + g * HP, o_addr = tmem + lane_base + 2 * HP + g * HP;
        uint8_t* pt = smem + SMEM_PT + g * PT_BYTES;
        bool ok = true;
        int tiles = 0, mine = 0;                                // running counts: key tiles of earlier items; key tiles this group has processed
        uint32_t exchanges = 0;                                 // completed phases of exchanged[g]
        // a warp's lanes have written `red`: the warp arrives once; then everybody waits (bounded) for the four warps
        auto exchange = [&]() -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars->exchanged[g]));
            return wait_bounded(smem_u32(&bars->exchanged[g]), (exchanges++) & 1, abort_flag, p.error_word, 740 + g);
        };

        for (int w = blockIdx.x; w < p.n_items && ok; w += gridDim.x) {
            const Item it = get_item(p, w);
            if (!it.valid) continue;
            const int j0 = g ^ (tiles & 1);                     // the group takes the tiles of its parity in the CTA's stream of tiles
            const int n_mine = it.n_kv > j0 ? (it.n_kv - j0 + 1) / 2 : 0;
            float m_run[HP], l_part[HP];
#pragma unroll
            for (int h = 0; h < HP; ++h) { m_run[h] = -INFINITY; l_part[h] = 0.f; }

            for (int jj = 0; jj < n_mine; ++jj, ++mine) {
                const int j = 2 * jj + j0, k0 = it.kv_base + j * BN;
                ok = wait_bounded(smem_u32(&bars->s_full[g]), mine & 1, abort_flag, p.error_word, 700 + g);
                if (!ok) break;
                tc_fence_after_sync();
                uint32_t sr[HP];
                tmem_ld16(s_addr, sr);
                tmem_wait_ld();
                const bool visible = k0 + key_in_tile < it.seq_kv;
                // the tile's maximum per head: over the warp's keys by integer reduction, over the four warps through shared memory
                float s[HP];
#pragma unroll
                for (int h = 0; h < HP; ++h) {
                    s[h] = visible ? __uint_as_float(sr[h]) : -INFINITY;
                    const int wmax = __reduce_max_sync(0xffffffffu, ordered(s[h]));
                    if (lane == h) bars->red[g][wq][h] = unordered(wmax);
                }
                ok = exchange();
                if (!ok) break;
                float alpha[HP];
                bool changed = false;
#pragma unroll
                for (int h = 0; h < HP; ++h) {
                    const float tile_max = fmaxf(fmaxf(bars->red[g][0][h], bars->red[g][1][h]), fmaxf(bars->red[g][2][h], bars->red[g][3][h]));
                    const float m_new = fmaxf(m_run[h], tile_max);
                    alpha[h] = fast_exp2((m_run[h] - m_new) * p.scale_log2);     // -inf - finite = -inf gives 0; equal maxima give 1
                    changed |= m_new != m_run[h];
                    m_run[h] = m_new;
                }
                uint32_t packed[HP / 2];
#pragma unroll
                for (int h = 0; h < HP; h += 2) {
                    const float p0 = fast_exp2((s[h] - m_run[h]) * p.scale_log2), p1 = fast_exp2((s[h + 1] - m_run[h + 1]) * p.scale_log2);
                    l_part[h] = l_part[h] * alpha[h] + p0;
                    l_part[h + 1] = l_part[h + 1] * alpha[h + 1] + p1;
                    packed[h / 2] = pack2<BF16>(p0, p1);
                }
                // the group's previous P^T V is through (always, once the first tile of the CTA is past): P^T may be
                // overwritten; inside an item O^T is rescaled when a maximum moved
                if (mine > 0) {
                    ok = wait_bounded(smem_u32(&bars->o_done[g]), (mine - 1) & 1, abort_flag, p.error_word, 710 + g);
                    if (!ok) break;
                    tc_fence_after_sync();
                    if (jj > 0 && changed) {                     // the same for every thread of the group: all hold the same maxima
                        uint32_t orow[HP];
                        tmem_ld16(o_addr, orow);
                        tmem_wait_ld();
#pragma unroll
                        for (int h = 0; h < HP; ++h) orow[h] = __float_as_uint(__uint_as_float(orow[h]) * alpha[h]);
                        tmem_st16(o_addr, orow);
                        tmem_wait_st();
                    }
                }
                // P^T[head][key] as 8-head x 8-key (16-byte) core matrices: 128 bytes apart along the keys, 2048 along the heads
#pragma unroll
                for (int h = 0; h < HP; h += 2) {
                    const uint32_t v = packed[h / 2];
                    uint8_t* at = pt + (h >> 3) * (BN * 16) + (key_in_tile >> 3) * 128 + (h & 7) * 16 + (key_in_tile & 7) * 2;
                    *reinterpret_cast<uint16_t*>(at) = (uint16_t)(v & 0xffffu);
                    *reinterpret_cast<uint16_t*>(at + 16) = (uint16_t)(v >> 16);
                }
                // value rows of slots nobody wrote (the sequence's last page): zero probabilities, but the bits there need not be numbers
                if (k0 + BN > it.seq_kv && (it.seq_kv & 15)) {
                    const int t = tiles + j, st = t % KV_STAGES;
                    ok = wait_bounded(smem_u32(&bars->v_full[st]), (t / KV_STAGES) & 1, abort_flag, p.error_word, 720 + g);
                    if (!ok) break;
                    const int first_row = it.seq_kv - k0, rows = 16 - (it.seq_kv & 15);
                    uint8_t* vt = smem + SMEM_V + st * TILE_BYTES;
                    for (int c = key_in_tile; c < rows * (D / 8); c += BM) {
                        const int r = first_row + c / (D / 8), piece = c % (D / 8);
                        *reinterpret_cast<uint4*>(vt + (piece >> 3) * (BN * 128) + r * 128 + (piece & 7) * 16) = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
                fence_proxy_async();
                tc_fence_before_sync();
                mbar_arrive(smem_u32(&bars->p_full[g]));
            }
            if (!ok) break;
            tiles += it.n_kv;

            // partial of this group for the combine kernel: per head the maximum (base-2 units), the sum, and O^T's column
            const long long part0 = ((long long)it.si * p.parts + 2 * it.chunk + g) * p.q_heads + (long long)it.kvh * G;
            if (n_mine > 0) {
                ok = wait_bounded(smem_u32(&bars->o_done[g]), (mine - 1) & 1, abort_flag, p.error_word, 730 + g);
                if (!ok) break;
                tc_fence_after_sync();
                uint32_t orow[HP];
                tmem_ld16(o_addr, orow);                         // lane = element of the head dimension
                tmem_wait_ld();
                tc_fence_before_sync();
#pragma unroll
                for (int h = 0; h < HP; ++h)
                    if (h < G) p.part_o[(part0 + h) * D + key_in_tile] = __uint_as_float(orow[h]);
                // the sums: over the warp's keys by shuffles, over the warps through shared memory
#pragma unroll
                for (int h = 0; h < HP; ++h) {
                    float v = l_part[h];
#pragma unroll
                    for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
                    if (lane == h) bars->red[g][wq][h] = v;
                }
                ok = exchange();
                if (!ok) break;
                if (wq == 0 && lane < G) {
                    const float l = bars->red[g][0][lane] + bars->red[g][1][lane] + bars->red[g][2][lane] + bars->red[g][3][lane];
                    float m = 0.f;
#pragma unroll
                    for (int h = 0; h < HP; ++h) m = lane == h ? m_run[h] : m;
                    p.part_ml[part0 + lane] = make_float2(m * p.scale_log2, l);
                }
                // the sums must be read before the next item's maxima overwrite them
                ok = exchange();
                if (!ok) break;
            } else if (wq == 0 && lane < G) {
                p.part_ml[part0 + lane] = make_float2(-INFINITY, 0.f);          // a one-tile chunk leaves group 1 nothing
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (warp == MMA_WARP) tmem_dealloc(tmem, TMEM_DECODE_COLS);
}

template <bool BF16>
ahpc_status launch_kernel(const PagedDecodeTcLaunch& a, const CUtensorMap& mq, const CUtensorMap& mv, const DecodeTcParams& p) {
    auto kernel = paged_decode_tc_kernel<BF16>;
    AHPC_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_TOTAL));
    // One CTA per item.  (The kernel can walk items w, w + gridDim.x, ... as one stream of tiles; a grid of one CTA per SM
    // doing so was measured slower - 230-260 us against 190-215 us on 64 sequences of 512..8192 tokens with 8 key/value
    // heads - although it no longer pays per item.)
    kernel<<<(unsigned)p.n_items, TC_THREADS, SMEM_TOTAL, a.stream>>>(mq, mv, p);
    AHPC_CUDA_OK(cudaGetLastError());
    return AHPC_SUCCESS;
}

}  // namespace

bool decode_tc_keys_supported(const PagedDecodeTcLaunch& a) {
    return a.head_dim == D && a.q_heads / a.kv_heads <= HP && (a.dtype == AHPC_F16 || a.dtype == AHPC_BF16);
}

ahpc_status launch_decode_tc_keys(const PagedDecodeTcLaunch& a) {
    CUtensorMap mq, mv;
    const long long rows = (long long)a.n_seqs * a.q_heads;
    const int64_t qs[4] = {rows * a.head_dim, rows * a.head_dim, a.head_dim, 1};
    const int64_t vs[4] = {a.page_elems, 16ll * a.head_dim, a.head_dim, 1};
    AHPC_TRY(make_map(&mq, a.q, a.dtype, 1, 1, (int)rows, a.head_dim, qs, HP));
    AHPC_TRY(make_map(&mv, a.v_data, a.dtype, a.num_pages, a.kv_heads, 16, a.head_dim, vs, 16));
    DecodeTcParams p{};
    p.k_data = static_cast<const uint16_t*>(a.k_data);
    p.table = a.table; p.seq_ids = a.seqs_dev; p.seq_len = a.seq_len;
    p.part_o = a.part_o; p.part_ml = a.part_ml;
    p.page_elems = a.page_elems; p.max_pages = a.max_pages; p.q_heads = a.q_heads; p.group = a.q_heads / a.kv_heads;
    p.kv_heads = a.kv_heads; p.n_seqs = a.n_seqs; p.split = a.split; p.chunks = a.chunks; p.parts = 2 * a.chunks;
    if ((long long)a.chunks * a.kv_heads * a.n_seqs > 2147483647ll) return fail(AHPC_UNSUPPORTED_OPERATION, "decode: too many chunks");
    p.n_items = a.chunks * a.kv_heads * a.n_seqs;
    p.scale_log2 = a.scale * 1.4426950408889634f;
    AHPC_TRY(error_word_for(a.device, &p.error_word));
    return a.dtype == AHPC_BF16 ? launch_kernel<true>(a, mq, mv, p) : launch_kernel<false>(a, mq, mv, p);
}

}  // namespace ahpc
