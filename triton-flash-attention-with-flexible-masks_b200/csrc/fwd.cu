// Forward kernel: O = softmax(mask(Q K^T * sm_scale)) V and the row log-sum-exp.
// Replaces `_fwd_kernel` (flash_triton.py:25-141). Same mathematics (base-2 online softmax,
// P rounded to the input dtype before P*V, fp32 accumulation), except that the scale is
// applied in fp32 to the fp32 scores instead of being folded into a rounded Q
// (flash_triton.py:88), and tiles the mask plan proves empty are not visited at all.
//
// Persistent: one CTA per SM walks work items (one item = one block of 128 queries of one
// (batch, head)); items are handed out in an order that puts the query blocks of
// all heads side by side, so that the CTAs of one round carry almost equal work. With document
// masks most items hold only a few tiles, so everything around the tiles is overlapped with the
// neighbouring items: a scheduler warp prepares the next item's tile list, the producer prefetches
// its Q / K / V, and the output tile leaves through an asynchronous TMA store.
//
// 12 warps:
//   warps 0-3  softmax group 0, warps 4-7 softmax group 1 (thread r of a group owns row r)
//   warp 8     TMA producer (Q per item, K and V rings that run across items)
//   warps 9,10 tcgen05.mma issuers, one per softmax group; warp 9 owns the TMEM allocation
//   warp 11    item scheduler: decodes the item, classifies its candidate tiles from the mask plan
//              and compacts the visited ones into a list in shared memory (two item slots)
// Visited key tiles alternate between the two groups: the CTA's g-th tile (counted across its items)
// uses score buffer S[g&1] and accumulates into O[g&1] with the group's own running max / sum for
// the item; the two partial results are merged in the item's epilogue, the chain of the item's even
// tiles first, so that the result does not depend on which group that was. Counting across items
// keeps every K / V ring slot (slot g % NS, NS even) with one issuer, which waits for each of
// its phases in turn, and lets consecutive one-tile items overlap on the two chains. TMEM columns: S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [256+D,256+2D).
// P (input dtype, two values per column) overwrites the first 64 columns of its S buffer.
#include <type_traits>
#include "common.cuh"
#include "params.cuh"

namespace fa {

constexpr int kTurnMinTiles = 8;  // items with fewer visited tiles do not serialise their exp phases

template <int D>
struct FwdSmem {
    static constexpr int NS = (D == 128) ? 2 : 4;  // depth of the K ring and of the V ring
    static constexpr int TILE = kBlk * D * 2;
    static constexpr int BOX = kBlk * 64 * 2;
    static constexpr int NBOX = D / 64;
    static constexpr int NKC = 8;  // depth of the key-code ring
    static constexpr int off_q = 0;  // two Q tiles; a slot also stages its item's O tile for the TMA store
    static constexpr int off_k = 2 * TILE;
    static constexpr int off_v = off_k + NS * TILE;
    static constexpr int off_list = off_v + NS * TILE;         // uint16 [2][kListCap]
    static constexpr int off_qc = off_list + 2 * kListCap * 2;  // int32  [2][128] query codes
    static constexpr int off_kc = off_qc + 2 * kBlk * 4;        // int32  [NKC][128] key codes, loaded with K on K's barrier
    static constexpr int off_ml = off_kc + NKC * kBlk * 4;      // float  [2][2 groups][m, l][128]
    static constexpr int off_info = off_ml + 2 * 2 * 2 * kBlk * 4;  // int32 [2][8]: T, lo, item (-1: no more items), -, query block, head, batch
    static constexpr int off_bar = off_info + 64;
    // item_full[2] item_empty[2] q_full[2] o_staged[2] k_full[NS] k_empty[NS] v_full[NS] v_empty[NS]
    // s_full[2] p_half0[2] p_half1[2] pv_done[2] turn[2] o_free[2] ml_full
    static constexpr int n_bar = 8 + 4 * NS + 12 + 1;
    static constexpr int off_misc = off_bar + n_bar * 8;  // tmem slot, abort flag
    static constexpr int total = off_misc + 16;
};

template <int D, bool BF16>
__global__ void __launch_bounds__(kAttnThreads, 1)
fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
           const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, const FwdParams p) {
    using S = FwdSmem<D>;
    constexpr int NS = S::NS;
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const MaskArgs& mk = p.mask;
    const int nQ = mk.L.nQ;
    const int HB = p.H * p.B;
    const int n_items = nQ * HB;
    unsigned int* ctr = mk.ctr ? mk.ctr + CTR_FWD : nullptr;

    volatile int* misc = reinterpret_cast<volatile int*>(smem + S::off_misc);  // [0] tmem, [1] abort
    volatile int* info = reinterpret_cast<volatile int*>(smem + S::off_info);
    const uint32_t bar0 = sbase + S::off_bar;
    auto BAR = [&](int i) { return bar0 + 8u * uint32_t(i); };
    constexpr int B_ITEMFULL = 0, B_ITEMEMPTY = 2, B_QFULL = 4, B_OSTAGED = 6, B_KFULL = 8, B_KEMPTY = 8 + NS,
                  B_VFULL = 8 + 2 * NS, B_VEMPTY = 8 + 3 * NS, B_SFULL = 8 + 4 * NS, B_PHALF0 = B_SFULL + 2,
                  B_PHALF1 = B_SFULL + 4, B_PVDONE = B_SFULL + 6, B_TURN = B_SFULL + 8, B_OFREE = B_SFULL + 10, B_MLFULL = B_SFULL + 12;
    Abort ab{misc + 1, p.status, p.wait_limit};

    if (tid == 0) {
        for (int s = 0; s < 2; ++s) {
            mbar_init(BAR(B_ITEMFULL + s), 1);
            mbar_init(BAR(B_ITEMEMPTY + s), 5);  // producer, two MMA issuers, one thread of each softmax group
            mbar_init(BAR(B_QFULL + s), 1);
            mbar_init(BAR(B_OSTAGED + s), 256);
            mbar_init(BAR(B_SFULL + s), 1);
            mbar_init(BAR(B_PHALF0 + s), 128);
            mbar_init(BAR(B_PHALF1 + s), 128);
            mbar_init(BAR(B_PVDONE + s), 1);
            mbar_init(BAR(B_TURN + s), 128);
            mbar_init(BAR(B_OFREE + s), 256);
        }
        mbar_init(BAR(B_MLFULL), 256);
        for (int s = 0; s < NS; ++s) {
            mbar_init(BAR(B_KFULL + s), 1);
            mbar_init(BAR(B_KEMPTY + s), 1);
            mbar_init(BAR(B_VFULL + s), 1);
            mbar_init(BAR(B_VEMPTY + s), 1);
        }
        misc[1] = (status_is_fatal(*reinterpret_cast<volatile int*>(p.status)) || (sbase & 1023u) != 0) ? 1 : 0;
        fence_mbar_init();
    }
    if (warp == 9) {
        tmem_alloc(sbase + S::off_misc, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = uint32_t(misc[0]);
    const bool aborted = misc[1] != 0;
    // an earlier launch on this device ran into a time-out that the host has not yet cleared
    if (aborted && (sbase & 1023u) == 0) nan_fill_outputs(smem + S::off_q, S::NBOX, &tmO, nullptr, nQ, p.H, p.B);

    auto sQ = [&](int s) { return sbase + S::off_q + uint32_t(s) * S::TILE; };
    auto sK = [&](int s) { return sbase + S::off_k + uint32_t(s) * S::TILE; };
    auto sV = [&](int s) { return sbase + S::off_v + uint32_t(s) * S::TILE; };
    auto list_of = [&](int s) { return reinterpret_cast<const uint16_t*>(smem + S::off_list) + s * kListCap; };
    // item -> (query block, head, batch). Heads are taken in groups of p.gh; inside a group the query
    // blocks go from the last one down (with a causal mask: long ones first) and the heads of the
    // group vary fastest. The CTAs thus work on neighbouring query blocks of a few heads at a time:
    // few enough that their K / V streams stay in L2, enough that not all CTAs pull the same lines.
    auto decode = [&](int j, int& qb, int& h, int& b) {
        const int per = p.gh * nQ;                 // items of a full group of heads
        const int grp = j / per, rem = j - grp * per;
        const int gsz = min(p.gh, HB - grp * p.gh);  // heads in this group (the last one may be smaller)
        const int pos = rem / gsz, bh = grp * p.gh + (rem - pos * gsz);
        b = bh / p.H;
        h = bh - b * p.H;
        // few items per CTA: longest first (sorted in the plan), so that no long item is left for the end
        qb = p.by_length ? mk.plan[mk.L.off_ordq + (int64_t(b) * mk.He + (mk.He == 1 ? 0 : h)) * nQ + pos] : nQ - 1 - pos;
    };

    if (warp >= 8) {
        setmaxnreg_dec<72>();
        if (aborted) {
            // a previous kernel reported an error: do nothing
        } else if (warp == 11) {
            // ------------------------------ item scheduler ------------------------------
            // Items are handed out in order from a counter in the plan (any CTA takes the next one: the
            // work per item varies with the mask); without counters (no plan given) they are
            // dealt out round robin in alternating direction, which evens out their sorted lengths.
            bool ok = true;
            for (int k = 0;; ++k) {
                const int s = k & 1, use = k >> 1;
                if (use > 0) ok = mbar_wait(BAR(B_ITEMEMPTY + s), (use - 1) & 1, ab, ST_WAIT_TIMEOUT + 11);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                int j = 0;
                if (lane == 0) {
                    if (ctr) j = int(atomicAdd(ctr, 1u));
                    else j = k * int(gridDim.x) + ((k & 1) ? int(gridDim.x) - 1 - int(blockIdx.x) : int(blockIdx.x));
                }
                j = __shfl_sync(0xffffffffu, j, 0);
                if (j >= n_items) {  // end marker
                    if (lane == 0) {
                        info[s * 8 + 2] = -1;
                        mbar_arrive(BAR(B_ITEMFULL + s));
                    }
                    break;
                }
                int qb, h, b;
                decode(j, qb, h, b);
                const int he = (mk.He == 1) ? 0 : h;
                int lo, hi;
                kv_range(mk, b, he, qb, lo, hi);
                int n = hi - lo;
                if (n > kListCap) n = kListCap;  // the host refuses problems that could exceed the cap
                uint16_t* list = reinterpret_cast<uint16_t*>(smem + S::off_list) + s * kListCap;
                int T = 0;
                for (int base = 0; base < n; base += 32) {
                    const int i = base + lane;
                    const uint32_t f = (i < n) ? classify_from_plan(mk, b, he, qb, lo + i) : 0u;
                    const uint32_t m = __ballot_sync(0xffffffffu, (f & TILE_VISIT) != 0);
                    if (f & TILE_VISIT) list[T + __popc(m & ((1u << lane) - 1u))] = uint16_t(uint32_t(i) | (f << 10));
                    T += __popc(m);
                }
                int4 qc4 = make_int4(0, 0, 0, 0);
                if (mk.mode == 1)
                    qc4 = *reinterpret_cast<const int4*>(mk.plan + mk.L.off_qc + (int64_t(b) * mk.He + he) * mk.L.Mpad +
                                                         int64_t(qb) * kBlk + lane * 4);
                reinterpret_cast<int4*>(smem + S::off_qc)[s * 32 + lane] = qc4;
                if (lane == 0) {
                    info[s * 8 + 0] = T;
                    info[s * 8 + 1] = lo;
                    info[s * 8 + 2] = j;
                    info[s * 8 + 4] = qb;
                    info[s * 8 + 5] = h;
                    info[s * 8 + 6] = b;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(BAR(B_ITEMFULL + s));
            }
        } else if (warp == 8) {
            // ------------------------------ TMA producer ------------------------------
            if (lane == 0) {
                tma_prefetch_desc(&tmQ);
                tma_prefetch_desc(&tmK);
                tma_prefetch_desc(&tmV);
                bool ok = true;
                int k = 0, G = 0;  // G: tiles of all earlier items (the K / V rings run across items)
                // TMA store of the O tile the softmax groups staged in slot (kk & 1) for item kk
                int item_qb[2] = {0, 0}, item_h[2] = {0, 0}, item_b[2] = {0, 0};  // the items in the two slots
                auto store_o = [&](int kk) {
                    const int s = kk & 1;
                    if (!mbar_wait(BAR(B_OSTAGED + s), (kk >> 1) & 1, ab, ST_WAIT_TIMEOUT + 13)) return false;
                    const int qb = item_qb[s], h = item_h[s], b = item_b[s];
                    for (int x = 0; x < S::NBOX; ++x) tma_store_4d(&tmO, sQ(s) + x * S::BOX, x * 64, qb * kBlk, h, b);
                    tma_store_commit();
                    tma_store_wait_read();
                    return true;
                };
                for (;; ++k) {
                    const int s = k & 1, use = k >> 1;
                    ok = mbar_wait(BAR(B_ITEMFULL + s), use & 1, ab, ST_WAIT_TIMEOUT + 12);
                    if (!ok) break;
                    const int T = info[s * 8 + 0], lo = info[s * 8 + 1], j = info[s * 8 + 2];
                    if (j < 0) break;
                    const uint16_t* list = list_of(s);
                    const int qb = info[s * 8 + 4], h = info[s * 8 + 5], b = info[s * 8 + 6];
                    const int hk = h / p.G;
                    const int he = (mk.He == 1) ? 0 : h;
                    // the slot still holds the staged O tile of item k-2: send it off first
                    if (use > 0) ok = store_o(k - 2);
                    if (!ok) break;
                    item_qb[s] = qb; item_h[s] = h; item_b[s] = b;
                    mbar_expect_tx(BAR(B_QFULL + s), S::TILE);
                    for (int x = 0; x < S::NBOX; ++x)
                        tma_load_4d(sQ(s) + x * S::BOX, &tmQ, BAR(B_QFULL + s), x * 64, qb * kBlk, h, b);
                    for (int t = 0; t <= T && ok; ++t) {  // K runs one tile ahead of V
                        if (t < T) {
                            const int kb = lo + (list[t] & 1023);
                            const int g = G + t, st = g % NS, ug = g / NS;
                            if (ug > 0) ok = mbar_wait(BAR(B_KEMPTY + st), (ug - 1) & 1, ab, ST_WAIT_TIMEOUT + 1);
                            if (!ok) break;
                            // The tile's key codes travel with K: they land in a ring of NKC slots and complete on
                            // K's barrier, so whoever has seen S(g) (computed after that barrier) may read them.
                            // Slot g % NKC was last read by the softmax of tile g - NKC, which is over: this thread
                            // has already waited for the P*V of tile g - 2 - NS before issuing V(g - 2).
                            mbar_expect_tx(BAR(B_KFULL + st), S::TILE + (mk.mode == 1 ? kBlk * 4 : 0));
                            for (int x = 0; x < S::NBOX; ++x)
                                tma_load_4d(sK(st) + x * S::BOX, &tmK, BAR(B_KFULL + st), x * 64, kb * kBlk, hk, b);
                            if (mk.mode == 1)
                                bulk_load_1d(sbase + S::off_kc + (g % S::NKC) * (kBlk * 4),
                                             mk.plan + mk.L.off_kc + (int64_t(b) * mk.He + he) * mk.L.Npad + int64_t(kb) * kBlk,
                                             kBlk * 4, BAR(B_KFULL + st));
                        }
                        if (t >= 1) {
                            const int kb = lo + (list[t - 1] & 1023);
                            const int g = G + t - 1, st = g % NS, ug = g / NS;
                            if (ug > 0) ok = mbar_wait(BAR(B_VEMPTY + st), (ug - 1) & 1, ab, ST_WAIT_TIMEOUT + 2);
                            if (!ok) break;
                            mbar_expect_tx(BAR(B_VFULL + st), S::TILE);
                            for (int x = 0; x < S::NBOX; ++x)
                                tma_load_4d(sV(st) + x * S::BOX, &tmV, BAR(B_VFULL + st), x * 64, kb * kBlk, hk, b);
                        }
                    }
                    G += T;
                    if (ok) mbar_arrive(BAR(B_ITEMEMPTY + s));
                }
                // the last two items' tiles
                if (ok && k >= 2) ok = store_o(k - 2);
                if (ok && k >= 1) ok = store_o(k - 1);
                tma_store_wait_all();
            }
        } else {
            // ------------------------------ MMA issuers ------------------------------
            // One issuing thread per softmax group: warp 9 owns the CTA's even visited tiles (S0 / O0),
            // warp 10 the odd ones (S1 / O1). The two chains touch disjoint TMEM and only share the
            // K / V rings, so neither thread ever waits on the other group's softmax. Within a
            // chain the MMAs of P*V(t) and S(t+2) are issued back to back (the tensor pipe accepts
            // only a few MMAs ahead and needs ~200 clocks to refill once drained): what S(t+2)
            // needs from TMA is waited for before P(t) is.
            if (lane == 0) {
                const int w = warp - 9;
                constexpr uint32_t idesc_s = make_idesc(BF16, 128, 128, false, false);
                constexpr uint32_t idesc_pv = make_idesc(BF16, 128, D, false, true);
                constexpr uint64_t desc_v = desc_mn_major(S::BOX);
                const uint32_t tS = tmem + uint32_t(w) * 128u;
                const uint32_t tO = tmem + 256u + uint32_t(w) * uint32_t(D);
                bool ok = true;
                int k = 0, G = 0, cw = 0;  // cw: tiles this chain has finished (phases of its barriers)
                int kkw = 0;               // items in which this chain had tiles (phase of its o_free barrier)
                for (;; ++k) {
                    const int s = k & 1, use = k >> 1;
                    ok = mbar_wait(BAR(B_ITEMFULL + s), use & 1, ab, ST_WAIT_TIMEOUT + 12);
                    if (!ok) break;
                    const int T = info[s * 8 + 0];
                    if (info[s * 8 + 2] < 0) break;
                    ok = mbar_wait(BAR(B_QFULL + s), use & 1, ab, ST_WAIT_TIMEOUT + 3);
                    if (!ok) break;
                    const uint32_t q_tile = sQ(s);
                    auto k_ready = [&](int g) {
                        return mbar_wait(BAR(B_KFULL + (g % NS)), (g / NS) & 1, ab, ST_WAIT_TIMEOUT + 4);
                    };
                    auto s_mmas = [&](int g) {
                        const int st = g % NS;
#pragma unroll
                        for (int kk = 0; kk < D / 16; ++kk) {
                            const uint32_t off = uint32_t(kk >> 2) * S::BOX + uint32_t(kk & 3) * 32u;
                            umma_ss(tS, smem_desc_at(kDescKMajor, q_tile + off), smem_desc_at(kDescKMajor, sK(st) + off),
                                    idesc_s, kk > 0);
                        }
                        umma_commit(BAR(B_KEMPTY + st));
                        umma_commit(BAR(B_SFULL + w));
                    };
                    const int t0 = (G ^ w) & 1;  // this chain's first tile of the item: G + t0 has parity w
                    const int nmine = (T > t0) ? (T - t0 + 1) / 2 : 0;
                    if (nmine > 0) {
                        ok = k_ready(G + t0);
                        if (!ok) break;
                        tc_fence_after();
                        s_mmas(G + t0);
                    }
                    for (int i = 0; i < nmine && ok; ++i, ++cw) {
                        const int g = G + t0 + 2 * i, st = g % NS;
                        const bool more = i + 1 < nmine;
                        ok = mbar_wait(BAR(B_VFULL + st), (g / NS) & 1, ab, ST_WAIT_TIMEOUT + 5);
                        if (ok && more) ok = k_ready(g + 2);
                        // The first P*V of an item overwrites O: the epilogue of the previous item in which this
                        // chain had tiles must have read it. (The barrier counts those items only, on both
                        // sides: a chain without tiles in an item runs through it and must not find itself two
                        // phases behind, where a parity wait can no longer tell "not yet" from "done".)
                        if (ok && i == 0 && kkw > 0) ok = mbar_wait(BAR(B_OFREE + w), (kkw - 1) & 1, ab, ST_WAIT_TIMEOUT + 14);
                        if (ok) ok = mbar_wait(BAR(B_PHALF0 + w), cw & 1, ab, ST_WAIT_TIMEOUT + 6);
                        if (!ok) break;
                        tc_fence_after();
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk)
                            umma_ts(tO, tS + uint32_t(kk) * 8u, smem_desc_at(desc_v, sV(st) + uint32_t(kk) * 2048u), idesc_pv,
                                    (i > 0 || kk > 0) ? 1u : 0u);
                        ok = mbar_wait(BAR(B_PHALF1 + w), cw & 1, ab, ST_WAIT_TIMEOUT + 6);
                        if (!ok) break;
                        tc_fence_after();
#pragma unroll
                        for (int kk = 4; kk < 8; ++kk)
                            umma_ts(tO, tS + uint32_t(kk) * 8u, smem_desc_at(desc_v, sV(st) + uint32_t(kk) * 2048u), idesc_pv, 1u);
                        umma_commit(BAR(B_VEMPTY + st));
                        umma_commit(BAR(B_PVDONE + w));
                        if (more) s_mmas(g + 2);
                    }
                    G += T;
                    if (nmine > 0) ++kkw;
                    if (ok) mbar_arrive(BAR(B_ITEMEMPTY + s));
                }
            }
        }
        __syncwarp();
    } else {
        setmaxnreg_inc<216>();
        // ------------------------------ softmax groups ------------------------------
        // Every wait is a bounded mbarrier wait: a thread whose wait was given up (alive == false)
        // leaves the item loop at once, and nobody is left waiting for it for longer than the limit.
        const int w = warp >> 2;  // group
        const int r = tid & 127;  // row inside the block
        const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
        const float c = p.scale_log2;
        const uint32_t tS = tmem + lane_base + uint32_t(w) * 128u;
        const uint32_t tO = tmem + lane_base + 256u + uint32_t(w) * uint32_t(D);
        bool alive = !aborted;
        int k = 0, cw = 0;  // cw: tiles this group has finished (phases of its barriers)
        int nturn = 0;      // turns this group has taken (phase of its turn barrier)
        int G = 0;          // tiles of all earlier items (stage / phase of the K and V rings)
        for (; alive; ++k) {
            const int s = k & 1, use = k >> 1;
            alive = mbar_wait(BAR(B_ITEMFULL + s), use & 1, ab, ST_WAIT_TIMEOUT + 12);
            alive = __all_sync(0xffffffffu, alive);
            if (!alive) break;
            const int T = info[s * 8 + 0];
            const int lo = info[s * 8 + 1];
            const int j = info[s * 8 + 2];
            if (j < 0) break;
            const uint16_t* list = list_of(s);
            const int qb = info[s * 8 + 4], h = info[s * 8 + 5], b = info[s * 8 + 6];
            const int row = qb * kBlk + r;
            const int qc = reinterpret_cast<const int*>(smem + S::off_qc)[s * kBlk + r];
            float m_run = -INFINITY, l_run = 0.f;
            int n_my = 0;
            const int we = G & 1;   // the group that owns the item's even tiles
            const int t0 = w ^ we;  // this group's first tile of the item
            const int n_other = (t0 == 0) ? T / 2 : (T + 1) / 2;  // tiles of the other group
            // short items: both groups simply run side by side; long items: the exp phase is taken in turns
            const bool turns = T >= kTurnMinTiles;
            if (turns && t0 == 1 && alive) mbar_arrive(BAR(B_TURN + we));  // the owner of tile 0 takes the first turn

            for (int t = t0; t < T && alive; t += 2, ++n_my, ++cw) {
                const uint32_t entry = list[t];
                const uint32_t fl = entry >> 10;
                const int k0 = (lo + int(entry & 1023u)) * kBlk;
                alive = mbar_wait(BAR(B_SFULL + w), cw & 1, ab, ST_WAIT_TIMEOUT + 7);
                alive = __all_sync(0xffffffffu, alive);
                if (!alive) break;
                tc_fence_after();
                uint32_t sr[128];
#pragma unroll
                for (int q = 0; q < 4; ++q) tmem_ld32(tS + uint32_t(q) * 32u, sr + q * 32);
                tc_wait_ld();
                float* sc = reinterpret_cast<float*>(sr);

                if (fl & (TILE_BOUND | TILE_DOC)) {
                    // keep(x) = (x <= lim) & (qc >= 0 | kc[x] == qc). The compare + select per entry is
                    // ALU work that costs as much as the tile's MMAs, so it is done per 32-key chunk
                    // where possible: a chunk is kept or masked as a whole when it lies entirely on
                    // one side of the bound and (for monotone key codes) holds one single document.
                    int lim = kBlk - 1;
                    if (fl & TILE_BOUND) {
                        int jmax = mk.N - 1;
                        if (mk.causal) jmax = min(jmax, row + mk.gap);
                        lim = jmax - k0;
                    }
                    const bool doc = (fl & TILE_DOC) && qc < 0;  // a row with qc >= 0 passes the id check everywhere
                    const int* kcs = reinterpret_cast<const int*>(smem + S::off_kc + ((G + t) % S::NKC) * (kBlk * 4));
                    // (the key codes completed on K's barrier, before the S MMA whose result was just read)
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        int state = 0;  // this row in chunk q: 0 keep all, 1 mask all, 2 entry by entry
                        if (32 * q > lim) state = 1;
                        else if (32 * q + 31 > lim) state = 2;
                        if (doc && state != 1) {
                            if (fl & TILE_KMONO) {
                                const int kf = kcs[32 * q], kl = kcs[32 * q + 31];
                                if (kf != kl) state = 2;
                                else if (kf != qc) state = 1;
                            } else {
                                state = 2;
                            }
                        }
                        if (!__any_sync(0xffffffffu, state == 2)) {
                            if (state == 1) {
#pragma unroll
                                for (int x = 0; x < 32; ++x) sc[32 * q + x] = -INFINITY;
                            }
                        } else if (doc) {
                            const int4* kc4 = reinterpret_cast<const int4*>(kcs + 32 * q);
#pragma unroll
                            for (int u = 0; u < 8; ++u) {
                                const int4 kc = kc4[u];
                                const int x = 32 * q + 4 * u;
                                sc[x + 0] = (kc.x == qc && x + 0 <= lim) ? sc[x + 0] : -INFINITY;
                                sc[x + 1] = (kc.y == qc && x + 1 <= lim) ? sc[x + 1] : -INFINITY;
                                sc[x + 2] = (kc.z == qc && x + 2 <= lim) ? sc[x + 2] : -INFINITY;
                                sc[x + 3] = (kc.w == qc && x + 3 <= lim) ? sc[x + 3] : -INFINITY;
                            }
                        } else {
#pragma unroll
                            for (int x = 0; x < 32; ++x) sc[32 * q + x] = (32 * q + x <= lim) ? sc[32 * q + x] : -INFINITY;
                        }
                    }
                }
                float mxa[8];
#pragma unroll
                for (int a = 0; a < 8; ++a) mxa[a] = max3(sc[a], sc[8 + a], sc[16 + a]);
#pragma unroll
                for (int x = 24; x < 120; x += 16) {
#pragma unroll
                    for (int a = 0; a < 8; ++a) mxa[a] = max3(mxa[a], sc[x + a], sc[x + 8 + a]);
                }
#pragma unroll
                for (int a = 0; a < 8; ++a) mxa[a] = fmaxf(mxa[a], sc[120 + a]);
                const float mx = fmaxf(max3(mxa[0], mxa[1], mxa[2]), max3(max3(mxa[3], mxa[4], mxa[5]), mxa[6], mxa[7]));
                float m_new = fmaxf(m_run, mx);
                // lazy rescale: keep the old reference point while the new maximum is within 2^8 of it
                const bool need = (m_new - m_run) * c > 8.0f;
                if (!need) m_new = m_run;
                if (__any_sync(0xffffffffu, need)) {
                    const float alpha = need ? fast_exp2((m_run - m_new) * c) : 1.0f;
                    l_run *= alpha;
                    if (n_my > 0) {
                        alive = mbar_wait(BAR(B_PVDONE + w), (cw - 1) & 1, ab, ST_WAIT_TIMEOUT + 8);
                        alive = __all_sync(0xffffffffu, alive);
                        if (!alive) break;
                        tc_fence_after();
#pragma unroll
                        for (int q = 0; q < D / 32; ++q) {
                            uint32_t orr[32];
                            tmem_ld32(tO + uint32_t(q) * 32u, orr);
                            tc_wait_ld();
#pragma unroll
                            for (int x = 0; x < 32; ++x) orr[x] = __float_as_uint(__uint_as_float(orr[x]) * alpha);
                            tmem_st32(tO + uint32_t(q) * 32u, orr);
                        }
                        tc_wait_st();
                    }
                }
                m_run = m_new;
                const float mneg = (m_run == -INFINITY) ? 0.f : -m_run * c;
                // exp2(s*c - m*c) on packed pairs; P goes to TMEM in two halves so that the first four
                // k-steps of P*V can start while the second half is still being exponentiated.
                const uint64_t c2 = pack_f2(c, c), mneg2 = pack_f2(mneg, mneg);
                uint64_t lacc0 = pack_f2(0.f, 0.f), lacc1 = lacc0;
                // The exp phase is taken in turns (barriers turn[0], turn[1]; the owner of tile 0 first): left alone,
                // the groups fall into lockstep, exponentiate together at half MUFU rate each and then
                // queue their MMAs together, which halves the use of both pipes. In turns, one group
                // exponentiates while the other group's P*V and next S run on the tensor pipe.
                if (turns) {
                    alive = mbar_wait(BAR(B_TURN + w), nturn & 1, ab, ST_WAIT_TIMEOUT + 10);
                    alive = __all_sync(0xffffffffu, alive);
                    if (!alive) break;
                    ++nturn;
                }
                auto exp_half = [&](int half) {
#pragma unroll
                    for (int q = 2 * half; q < 2 * half + 2; ++q) {
                        uint32_t pk[16];
#pragma unroll
                        for (int x = 0; x < 16; ++x) {
                            const uint64_t x2 = fma_f2(pack_f2(sc[32 * q + 2 * x], sc[32 * q + 2 * x + 1]), c2, mneg2);
                            float x0, x1;
                            unpack_f2(x2, x0, x1);
                            const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
                            if (x & 1) lacc1 = add_f2(lacc1, pack_f2(p0, p1)); else lacc0 = add_f2(lacc0, pack_f2(p0, p1));
                            pk[x] = pack2<BF16>(p0, p1);
                        }
                        tmem_st16(tS + uint32_t(q) * 16u, pk);
                    }
                    tc_wait_st();
                    tc_fence_before();
                    mbar_arrive(BAR((half ? B_PHALF1 : B_PHALF0) + w));
                };
                exp_half(0);
                exp_half(1);
                // hand the turn over, unless the other group has no tile left to take it for
                if (turns && (t0 == 0 ? (n_my < n_other) : (n_my + 1 < n_other))) mbar_arrive(BAR(B_TURN + (w ^ 1)));
                {
                    float a0, a1, b0, b1;
                    unpack_f2(lacc0, a0, a1);
                    unpack_f2(lacc1, b0, b1);
                    l_run += (a0 + a1) + (b0 + b1);
                }
            }

            // ------------------------------ item epilogue ------------------------------
            // wait for this group's last P*V, then merge the two partial softmaxes
            if (!alive) break;
            if (T == 0) {
                // nobody has waited for this item's Q load yet, and its slot is about to become the staging
                // area of the (all-zero) output tile: the load must have landed first
                alive = mbar_wait(BAR(B_QFULL + s), use & 1, ab, ST_WAIT_TIMEOUT + 17);
                alive = __all_sync(0xffffffffu, alive);
                if (!alive) break;
            }
            if (n_my > 0) {
                alive = mbar_wait(BAR(B_PVDONE + w), (cw - 1) & 1, ab, ST_WAIT_TIMEOUT + 9);
                alive = __all_sync(0xffffffffu, alive);
                if (!alive) break;
            }
            float* ml = reinterpret_cast<float*>(smem + S::off_ml) + s * (4 * kBlk);  // [2 groups][m, l][128]
            ml[(w * 2 + 0) * kBlk + r] = m_run;
            ml[(w * 2 + 1) * kBlk + r] = l_run;
            tc_fence_before();
            mbar_arrive(BAR(B_MLFULL));  // both groups are past all MMAs of this item
            alive = mbar_wait(BAR(B_MLFULL), k & 1, ab, ST_WAIT_TIMEOUT + 16);
            alive = __all_sync(0xffffffffu, alive);
            if (!alive) break;
            tc_fence_after();
            // index 0: the chain of the item's even tiles, 1: of its odd tiles
            const float m0 = ml[(we * 2 + 0) * kBlk + r], l0 = ml[(we * 2 + 1) * kBlk + r];
            const float m1 = ml[((we ^ 1) * 2 + 0) * kBlk + r], l1 = ml[((we ^ 1) * 2 + 1) * kBlk + r];
            const float mt = fmaxf(m0, m1);
            const float a0 = (m0 == -INFINITY) ? 0.f : fast_exp2((m0 - mt) * c);
            const float a1 = (m1 == -INFINITY) ? 0.f : fast_exp2((m1 - mt) * c);
            const float lt = l0 * a0 + l1 * a1;
            const float inv = (lt > 0.f) ? 1.0f / lt : 0.f;
            const float f0 = a0 * inv, f1 = a1 * inv;
            const bool use0 = (T > 0) && (f0 != 0.f), use1 = (T > 1) && (f1 != 0.f);
            const bool healthy = alive && (misc[1] == 0);
            if (w == 0 && healthy) {
                const float lse = (lt > 0.f) ? fmaf(mt, c, log2f(lt)) : -INFINITY;
                p.lse[(int64_t(b) * p.H + h) * mk.L.Mpad + row] = lse;
            }
            // this thread's half row: columns [w*D/2, (w+1)*D/2) of both accumulators
            constexpr int HALF = D / 2;
            const uint32_t c0 = uint32_t(w) * HALF;
            uint32_t outw[HALF / 2];
#pragma unroll
            for (int q = 0; q < HALF / 32; ++q) {
                uint32_t x0[32], x1[32];
                // tcgen05.ld is warp-collective: always executed, the values are ignored when unused
                tmem_ld32(tmem + lane_base + 256u + uint32_t(we * D) + c0 + uint32_t(q) * 32u, x0);
                tmem_ld32(tmem + lane_base + 256u + uint32_t((we ^ 1) * D) + c0 + uint32_t(q) * 32u, x1);
                tc_wait_ld();
#pragma unroll
                for (int x = 0; x < 16; ++x) {
                    float v0 = 0.f, v1 = 0.f;
                    if (use0) {
                        v0 = __uint_as_float(x0[2 * x]) * f0;
                        v1 = __uint_as_float(x0[2 * x + 1]) * f0;
                    }
                    if (use1) {
                        v0 = fmaf(__uint_as_float(x1[2 * x]), f1, v0);
                        v1 = fmaf(__uint_as_float(x1[2 * x + 1]), f1, v1);
                    }
                    outw[16 * q + x] = pack2<BF16>(v0, v1);
                }
            }
            // both accumulators have been read: the MMA issuers may start the next item's P*V
            tc_fence_before();
            if (T > 0) mbar_arrive(BAR(B_OFREE + we));        // the chain of the even tiles had some
            if (T > 1) mbar_arrive(BAR(B_OFREE + (we ^ 1)));  // so had the other chain
            // Stage the O tile in this item's Q slot (Q is dead: every S MMA of the item has
            // completed) in the 128-byte-swizzled layout of the tensor map; the producer warp issues
            // the TMA store when every thread has arrived, and reuses the slot once it has been read.
            {
                uint8_t* stage = smem + S::off_q + s * S::TILE;
#pragma unroll
                for (int i = 0; i < HALF / 8; ++i) {
                    const int cg = int(c0) / 8 + i;  // 16-byte chunk of the row
                    const int box = cg >> 3, ch = cg & 7;
                    uint4* dst = reinterpret_cast<uint4*>(stage + box * S::BOX + r * 128 + ((ch ^ (r & 7)) << 4));
                    *dst = make_uint4(outw[4 * i], outw[4 * i + 1], outw[4 * i + 2], outw[4 * i + 3]);
                }
            }
            fence_proxy_async();
            if (healthy) mbar_arrive(BAR(B_OSTAGED + s));  // the producer warp issues the TMA store
            G += T;
            if (r == 0 && alive) mbar_arrive(BAR(B_ITEMEMPTY + s));
        }
    }

    // ------------------------------ tear-down ------------------------------
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
    // the last CTA to leave clears the work counters for the next launch that uses this plan
    if (tid == 0 && ctr) {
        __threadfence();
        if (atomicAdd(ctr + 1, 1u) == gridDim.x - 1) {
            ctr[0] = 0;
            ctr[1] = 0;
        }
    }
}

// ---- host launcher (called from api.cu) -------------------------------------------------
template <int D, bool BF16>
static cudaError_t launch_fwd_t(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                                const CUtensorMap& to, const FwdParams& p, int num_sms, cudaStream_t stream) {
    auto kern = fwd_kernel<D, BF16>;
    constexpr int smem = FwdSmem<D>::total;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    const int n_items = p.mask.L.nQ * p.H * p.B;
    dim3 grid(n_items < num_sms ? n_items : num_sms);
    kern<<<grid, kAttnThreads, smem, stream>>>(tq, tk, tv, to, p);
    return cudaGetLastError();
}


cudaError_t launch_fwd(int D, bool bf16, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                       const CUtensorMap& to, const FwdParams& p, int num_sms, cudaStream_t stream) {
    if (D == 128) return bf16 ? launch_fwd_t<128, true>(tq, tk, tv, to, p, num_sms, stream)
                              : launch_fwd_t<128, false>(tq, tk, tv, to, p, num_sms, stream);
    return bf16 ? launch_fwd_t<64, true>(tq, tk, tv, to, p, num_sms, stream)
                : launch_fwd_t<64, false>(tq, tk, tv, to, p, num_sms, stream);
}

}  // namespace fa
