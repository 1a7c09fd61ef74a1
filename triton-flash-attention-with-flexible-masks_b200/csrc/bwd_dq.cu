// dQ kernel. Replaces `_bwd_q_kernel` (flash_triton.py:323-431): per block of 128 queries,
// walk the visited key tiles, recompute P = exp2(S*scale*log2e - LSE), dP = dO V^T,
// dS = P * (dP - delta) with masked entries zeroed, dQ += dS K, and scale by sm_scale at the end.
//
// Persistent: min(items, SMs) CTAs, item = one query block of one (batch, head). 12 warps:
//   warps 0-7  two compute groups; thread r of group g owns query row r and key columns
//              [64g, 64g+64) of every tile
//   warp 8     TMA producer (per item Q with the per-row LSE / delta, and dO; K ring; V) and the TMA
//              store of a finished item's dQ
//   warp 9     tcgen05.mma issuer for S and dQ; owns the TMEM allocation
//   warp 10    tcgen05.mma issuer for dP
//   warp 11    scheduler: per item, the range of candidate key blocks and their codes
// Q has two slots (item parity); a slot also stages its item's dQ for the TMA store, so the next
// item's Q, K and first S tiles do not wait for the epilogue. dO, V and the dP columns are single
// buffers that are released early (after the last dP MMA, which runs a tile ahead of dQ).
// TMEM columns: S0 [0,128) S1 [128,256) dP [256,384) dQ [384,384+D). dS (input dtype) is
// written over the first half of each group's own S columns and fed to the dQ MMA from TMEM.
#include "common.cuh"
#include "params.cuh"

namespace fa {

template <int D>
struct DqSmem {
    static constexpr int NSK = (D == 128) ? 3 : 4;  // K(t) is read by S(t) and, a tile later, by dQ(t)
    static constexpr int TILE = kBlk * D * 2;
    static constexpr int BOX = kBlk * 64 * 2;
    static constexpr int NBOX = D / 64;
    static constexpr int VEC = 2 * kBlk * 4;    // lse, delta of one query block
    static constexpr int FLAGS = kListCap / 4;  // one item's candidate codes, 2 bits each
    static constexpr int off_q = 0;  // two slots
    static constexpr int off_do = 2 * TILE;
    static constexpr int off_v = 3 * TILE;
    static constexpr int off_k = 4 * TILE;
    static constexpr int off_vec = off_k + NSK * TILE;  // two slots
    static constexpr int off_flags = off_vec + 2 * VEC;  // two slots
    static constexpr int off_info = off_flags + 2 * FLAGS;  // two slots x {lo, n, tiles, item, query block, head, batch, -}
    static constexpr int off_bar = off_info + 64;
    // item_full[2], item_empty[2], q_full[2], staged[2], do_full, do_empty, v_full, v_empty, k_full[NSK],
    // k_empty[NSK], s_full[2], ds_full[2], dp_full, done, acc_free
    static constexpr int n_bar = 8 + 4 + 2 * NSK + 4 + 3;
    static constexpr int off_misc = off_bar + n_bar * 8;
    static constexpr int total = off_misc + 16;
};
static_assert(DqSmem<128>::total <= 232448 && DqSmem<64>::total <= 232448, "shared memory budget");

// Per-candidate code kept in shared memory (2 bits): 0 not visited, 1 visited without id check,
// 2 id check. Whether a tile needs the bound check (key tail, causal diagonal) follows from its
// coordinates alone.
enum : uint32_t { QC_SKIP = 0u, QC_PLAIN = 1u, QC_DOC = 2u };

struct DqWalk {
    const uint8_t* fl;
    int n;
    __device__ __forceinline__ uint32_t code(int c) const { return (uint32_t(fl[c >> 2]) >> (2 * (c & 3))) & 3u; }
    __device__ __forceinline__ int first_from(int c) const {
        while (c < n && code(c) == QC_SKIP) ++c;
        return c;
    }
};

template <int D, bool BF16>
__global__ void __launch_bounds__(kAttnThreads, 1)
bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
              const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
              const __grid_constant__ CUtensorMap tmdQ, const DqParams p) {
    using S = DqSmem<D>;
    constexpr int NSK = S::NSK;
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const MaskArgs& mk = p.mask;
    const int nQ = mk.L.nQ;
    const int HB = p.H * p.B;
    const int n_items = nQ * HB;
    unsigned int* ctr = mk.ctr ? mk.ctr + CTR_DQ : nullptr;
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

    volatile int* misc = reinterpret_cast<volatile int*>(smem + S::off_misc);
    volatile int* info = reinterpret_cast<volatile int*>(smem + S::off_info);
    const uint32_t bar0 = sbase + S::off_bar;
    auto BAR = [&](int i) { return bar0 + 8u * uint32_t(i); };
    constexpr int B_ITEMFULL = 0, B_ITEMEMPTY = 2, B_QFULL = 4, B_STAGED = 6, B_DOFULL = 8, B_DOEMPTY = 9, B_VFULL = 10,
                  B_VEMPTY = 11, B_KFULL = 12, B_KEMPTY = 12 + NSK, B_SFULL = 12 + 2 * NSK, B_DSFULL = B_SFULL + 2,
                  B_DPFULL = B_SFULL + 4, B_DONE = B_SFULL + 5, B_ACCFREE = B_SFULL + 6;
    Abort ab{misc + 1, p.status, p.wait_limit};

    auto sQ = [&](int s) { return sbase + S::off_q + uint32_t(s) * S::TILE; };
    const uint32_t sdO = sbase + S::off_do, sV = sbase + S::off_v;
    auto sK = [&](int s) { return sbase + S::off_k + uint32_t(s) * S::TILE; };
    auto sVec = [&](int s) { return sbase + S::off_vec + uint32_t(s) * S::VEC; };
    auto walk_of = [&](int s, int n) { return DqWalk{smem + S::off_flags + s * S::FLAGS, n}; };

    if (tid == 0) {
        for (int s = 0; s < 2; ++s) {
            mbar_init(BAR(B_ITEMFULL + s), 1);
            mbar_init(BAR(B_ITEMEMPTY + s), 11);  // producer, two MMA issuers, eight compute warps
            mbar_init(BAR(B_QFULL + s), 1);
            mbar_init(BAR(B_STAGED + s), 256);
            mbar_init(BAR(B_SFULL + s), 1);
            mbar_init(BAR(B_DSFULL + s), 256);
        }
        mbar_init(BAR(B_DOFULL), 1); mbar_init(BAR(B_DOEMPTY), 1);
        mbar_init(BAR(B_VFULL), 1); mbar_init(BAR(B_VEMPTY), 1);
        for (int s = 0; s < NSK; ++s) { mbar_init(BAR(B_KFULL + s), 1); mbar_init(BAR(B_KEMPTY + s), 1); }
        mbar_init(BAR(B_DPFULL), 1);
        mbar_init(BAR(B_DONE), 1);
        mbar_init(BAR(B_ACCFREE), 256);
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
    if (aborted && (sbase & 1023u) == 0) nan_fill_outputs(smem + S::off_q, S::NBOX, &tmdQ, nullptr, nQ, p.H, p.B);

    if (warp >= 8) {
        setmaxnreg_dec<56>();
        if (aborted) {
        } else if (warp == 11) {
            // ------------------------------ scheduler ------------------------------
            // Item k goes to slot k & 1: range [lo, lo + n) of candidate key blocks, a 2-bit code per
            // candidate, the number of visited tiles, the item index (-1: no more items). Items are
            // handed out in order from a counter in the plan (any CTA takes the next one: the work
            // per item varies with the mask); without counters (no plan given) they are dealt out
            // round robin in alternating direction, which evens out their sorted lengths.
            bool ok = true;
            for (int k = 0;; ++k) {
                const int s = k & 1, use = k >> 1;
                if (use > 0) ok = mbar_wait(BAR(B_ITEMEMPTY + s), (use - 1) & 1, ab, ST_WAIT_TIMEOUT + 31);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                int j = 0;
                if (lane == 0) {
                    if (ctr) j = int(atomicAdd(ctr, 1u));
                    else j = k * int(gridDim.x) + ((k & 1) ? int(gridDim.x) - 1 - int(blockIdx.x) : int(blockIdx.x));
                }
                j = __shfl_sync(0xffffffffu, j, 0);
                if (j >= n_items) {
                    if (lane == 0) {
                        info[s * 8 + 3] = -1;
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
                uint8_t* fl = smem + S::off_flags + s * S::FLAGS;
                int cnt = 0;
                for (int i = lane; 4 * i < n; i += 32) {
                    uint32_t byte = 0;
                    for (int e = 0; e < 4; ++e) {
                        const int c = 4 * i + e;
                        if (c >= n) break;
                        const uint32_t f = classify_from_plan(mk, b, he, qb, lo + c);
                        const uint32_t code = !(f & TILE_VISIT) ? QC_SKIP : (f & TILE_DOC) ? QC_DOC : QC_PLAIN;
                        cnt += (code != QC_SKIP);
                        byte |= code << (2 * e);
                    }
                    fl[i] = uint8_t(byte);
                }
                for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
                __syncwarp();
                if (lane == 0) {
                    info[s * 8 + 0] = lo;
                    info[s * 8 + 1] = n;
                    info[s * 8 + 2] = cnt;
                    info[s * 8 + 3] = j;
                    info[s * 8 + 4] = qb;
                    info[s * 8 + 5] = h;
                    info[s * 8 + 6] = b;
                    mbar_arrive(BAR(B_ITEMFULL + s));
                }
            }
        } else if (warp == 8) {
            // ------------------------------ TMA producer ------------------------------
            if (lane == 0) {
                tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmdO); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
                tma_prefetch_desc(&tmdQ);
                bool ok = true;
                int k = 0, kk = 0;  // items, items with tiles
                int gt = 0;         // tiles of all earlier items (stage / phase of the K ring and of V)
                int item_qb[2] = {0, 0}, item_h[2] = {0, 0}, item_b[2] = {0, 0};  // the items in the two slots
                // TMA store of the dQ tile the compute groups staged in slot (i & 1) for item i
                auto store_dq = [&](int i) {
                    const int s = i & 1;
                    if (!mbar_wait(BAR(B_STAGED + s), (i >> 1) & 1, ab, ST_WAIT_TIMEOUT + 32)) return false;
                    if (misc[1] == 0) {
                        const int qb = item_qb[s], h = item_h[s], b = item_b[s];
                        for (int x = 0; x < S::NBOX; ++x) tma_store_4d(&tmdQ, sQ(s) + x * S::BOX, x * 64, qb * kBlk, h, b);
                        tma_store_commit();
                        tma_store_wait_read();
                    }
                    return true;
                };
                for (;; ++k) {
                    const int s = k & 1;
                    ok = mbar_wait(BAR(B_ITEMFULL + s), (k >> 1) & 1, ab, ST_WAIT_TIMEOUT + 33);
                    if (!ok) break;
                    const int lo = info[s * 8 + 0], n = info[s * 8 + 1], T = info[s * 8 + 2], j = info[s * 8 + 3];
                    if (j < 0) break;
                    const int qb = info[s * 8 + 4], h = info[s * 8 + 5], b = info[s * 8 + 6];
                    const int hk = h / p.G;
                    // the slot still holds the staged dQ tile of item k-2: send it off first
                    if (k >= 2) ok = store_dq(k - 2);
                    if (!ok) break;
                    item_qb[s] = qb; item_h[s] = h; item_b[s] = b;
                    // Q with the rows' LSE and delta (also for an item without tiles: its dQ = 0 is staged in the slot)
                    mbar_expect_tx(BAR(B_QFULL + s), S::TILE + S::VEC);
                    for (int x = 0; x < S::NBOX; ++x)
                        tma_load_4d(sQ(s) + x * S::BOX, &tmQ, BAR(B_QFULL + s), x * 64, qb * kBlk, h, b);
                    const int64_t roff = (int64_t(b) * p.H + h) * mk.L.Mpad + int64_t(qb) * kBlk;
                    bulk_load_1d(sVec(s), p.lse + roff, kBlk * 4, BAR(B_QFULL + s));
                    bulk_load_1d(sVec(s) + kBlk * 4, p.delta + roff, kBlk * 4, BAR(B_QFULL + s));
                    if (T > 0) {
                        const DqWalk wk = walk_of(s, n);
                        int ck = wk.first_from(0), cv = ck;  // cursors of the K and of the V stream
                        for (int t = 0; t <= T && ok; ++t) {  // K runs one tile ahead of V
                            if (t < T) {
                                const int gi = gt + t, st = gi % NSK, use = gi / NSK;
                                if (use > 0) ok = mbar_wait(BAR(B_KEMPTY + st), (use - 1) & 1, ab, ST_WAIT_TIMEOUT + 21);
                                if (!ok) break;
                                mbar_expect_tx(BAR(B_KFULL + st), S::TILE);
                                for (int x = 0; x < S::NBOX; ++x)
                                    tma_load_4d(sK(st) + x * S::BOX, &tmK, BAR(B_KFULL + st), x * 64, (lo + ck) * kBlk, hk, b);
                                ck = wk.first_from(ck + 1);
                            }
                            if (t == 0) {
                                // dO once the previous item's last dP MMA has read the tile
                                if (kk > 0) ok = mbar_wait(BAR(B_DOEMPTY), (kk - 1) & 1, ab, ST_WAIT_TIMEOUT + 34);
                                if (!ok) break;
                                mbar_expect_tx(BAR(B_DOFULL), S::TILE);
                                for (int x = 0; x < S::NBOX; ++x)
                                    tma_load_4d(sdO + x * S::BOX, &tmdO, BAR(B_DOFULL), x * 64, qb * kBlk, h, b);
                            } else {
                                const int gi = gt + t - 1;
                                if (gi > 0) ok = mbar_wait(BAR(B_VEMPTY), (gi - 1) & 1, ab, ST_WAIT_TIMEOUT + 22);
                                if (!ok) break;
                                mbar_expect_tx(BAR(B_VFULL), S::TILE);
                                for (int x = 0; x < S::NBOX; ++x)
                                    tma_load_4d(sV + x * S::BOX, &tmV, BAR(B_VFULL), x * 64, (lo + cv) * kBlk, hk, b);
                                cv = wk.first_from(cv + 1);
                            }
                        }
                        if (!ok) break;
                        gt += T;
                        ++kk;
                    }
                    mbar_arrive(BAR(B_ITEMEMPTY + s));
                }
                // the last two items' tiles
                if (ok && k >= 2) ok = store_dq(k - 2);
                if (ok && k >= 1) ok = store_dq(k - 1);
            }
        } else {
            // ------------------------------ MMA issuers (warps 9, 10) ------------------------------
            // Two issuing threads, so that the blocking tcgen05.mma issue and barrier round trips of
            // one stream do not delay the other:
            //   warp 9 : S(0), S(1); then per tile dQ(t) += dS K(t) followed by S(t+2) (which
            //            overwrites dS(t): same thread, in order)
            //   warp 10: dP(t+1) = dO V(t+1)^T as soon as dS(t) has been written (dP columns free)
            // Tiles are numbered across items (gi), so that the S buffers, the K ring, V and every
            // per-tile barrier simply carry on from one item to the next.
            if (lane == 0) {
                constexpr uint32_t idesc_s = make_idesc(BF16, 128, 128, false, false);
                constexpr uint32_t idesc_dq = make_idesc(BF16, 128, D, false, true);
                constexpr uint64_t desc_mn = desc_mn_major(S::BOX);
                auto k_ready = [&](int gi) { return mbar_wait(BAR(B_KFULL + gi % NSK), (gi / NSK) & 1, ab, ST_WAIT_TIMEOUT + 24); };
                auto ss_mmas = [&](uint32_t d, uint32_t a_tile, uint32_t b_tile) {
#pragma unroll
                    for (int kk2 = 0; kk2 < D / 16; ++kk2) {
                        const uint32_t off = uint32_t(kk2 >> 2) * S::BOX + uint32_t(kk2 & 3) * 32u;
                        umma_ss(d, smem_desc_at(kDescKMajor, a_tile + off), smem_desc_at(kDescKMajor, b_tile + off),
                                idesc_s, kk2 > 0);
                    }
                };
                bool ok = true;
                int k = 0, kk = 0, gt = 0;
                for (;; ++k) {
                    const int s = k & 1;
                    ok = mbar_wait(BAR(B_ITEMFULL + s), (k >> 1) & 1, ab, ST_WAIT_TIMEOUT + 33);
                    if (!ok) break;
                    const int T = info[s * 8 + 2];
                    if (info[s * 8 + 3] < 0) break;
                    if (T > 0 && warp == 9) {
                        ok = mbar_wait(BAR(B_QFULL + s), (k >> 1) & 1, ab, ST_WAIT_TIMEOUT + 23);
                        const uint32_t q_tile = sQ(s);
                        for (int t = 0; t < 2 && t < T && ok; ++t) {
                            const int gi = gt + t;
                            ok = k_ready(gi);
                            if (ok) {
                                tc_fence_after();
                                ss_mmas(tmem + uint32_t(gi & 1) * 128u, q_tile, sK(gi % NSK));
                                umma_commit(BAR(B_SFULL + (gi & 1)));
                            }
                        }
                        // dQ(0) overwrites the accumulator: the previous item's epilogue must have read it
                        if (ok && kk > 0) ok = mbar_wait(BAR(B_ACCFREE), (kk - 1) & 1, ab, ST_WAIT_TIMEOUT + 35);
                        for (int t = 0; t < T && ok; ++t) {
                            const int gi = gt + t, st = gi % NSK;
                            ok = mbar_wait(BAR(B_DSFULL + (gi & 1)), (gi >> 1) & 1, ab, ST_WAIT_TIMEOUT + 26);
                            if (!ok) break;
                            tc_fence_after();
                            const uint32_t a = tmem + uint32_t(gi & 1) * 128u;
#pragma unroll
                            for (int kk2 = 0; kk2 < kBlk / 16; ++kk2) {
                                const uint32_t acol = (kk2 < 4) ? uint32_t(kk2) * 8u : 64u + uint32_t(kk2 - 4) * 8u;
                                umma_ts(tmem + 384u, a + acol, smem_desc_at(desc_mn, sK(st) + uint32_t(kk2) * 2048u), idesc_dq,
                                        (t > 0 || kk2 > 0) ? 1u : 0u);
                            }
                            umma_commit(BAR(B_KEMPTY + st));
                            // K(t+2) reuses the stage that dQ(t-1) releases, so it is waited for only now
                            if (t + 2 < T) {
                                ok = k_ready(gi + 2);
                                if (ok) {
                                    tc_fence_after();
                                    ss_mmas(a, q_tile, sK((gi + 2) % NSK));
                                    umma_commit(BAR(B_SFULL + (gi & 1)));
                                }
                            }
                        }
                        if (!ok) break;
                        umma_commit(BAR(B_DONE));
                    } else if (T > 0) {
                        ok = mbar_wait(BAR(B_DOFULL), kk & 1, ab, ST_WAIT_TIMEOUT + 23);
                        for (int t = 0; t < T && ok; ++t) {
                            const int gi = gt + t;
                            ok = mbar_wait(BAR(B_VFULL), gi & 1, ab, ST_WAIT_TIMEOUT + 25);
                            // dP(gi) may overwrite the dP columns once every thread has read dP(gi-1)
                            if (ok && gi > 0) ok = mbar_wait(BAR(B_DSFULL + ((gi - 1) & 1)), ((gi - 1) >> 1) & 1, ab, ST_WAIT_TIMEOUT + 26);
                            if (!ok) break;
                            tc_fence_after();
                            ss_mmas(tmem + 256u, sdO, sV);
                            umma_commit(BAR(B_VEMPTY));
                            umma_commit(BAR(B_DPFULL));
                        }
                        if (!ok) break;
                        umma_commit(BAR(B_DOEMPTY));
                    }
                    if (T > 0) ++kk;
                    gt += T;
                    mbar_arrive(BAR(B_ITEMEMPTY + s));
                }
            }
        }
        __syncwarp();
    } else {
        setmaxnreg_inc<224>();
        // ------------------------------ compute groups ------------------------------
        const int w = warp >> 2;
        const int r = tid & 127;
        const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
        const int cbase = 64 * w;
        const float c = p.scale_log2;
        bool ok = !aborted;
        int k = 0, kk = 0, gt = 0;
        for (; ok; ++k) {
            const int s = k & 1;
            ok = mbar_wait(BAR(B_ITEMFULL + s), (k >> 1) & 1, ab, ST_WAIT_TIMEOUT + 33);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const int lo = info[s * 8 + 0], n = info[s * 8 + 1], T = info[s * 8 + 2], j = info[s * 8 + 3];
            if (j < 0) break;
            const int qb = info[s * 8 + 4], h = info[s * 8 + 5], b = info[s * 8 + 6];
            const int he = (mk.He == 1) ? 0 : h;
            const DqWalk wk = walk_of(s, n);
            const int row = qb * kBlk + r;
            const int q0 = qb * kBlk;
            const int64_t bh_ids = int64_t(b) * mk.He + he;
            const int qc = (mk.mode == 1) ? __ldg(mk.plan + mk.L.off_qc + bh_ids * mk.L.Mpad + row) : 0;
            // Q's barrier also covers the rows' LSE and delta; the slot is this item's staging area later
            ok = mbar_wait(BAR(B_QFULL + s), (k >> 1) & 1, ab, ST_WAIT_TIMEOUT + 36);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const float lse = reinterpret_cast<const float*>(smem + S::off_vec + s * S::VEC)[r];
            const float delta = reinterpret_cast<const float*>(smem + S::off_vec + s * S::VEC)[kBlk + r];

            int cc = wk.first_from(0);
            for (int t = 0; t < T && ok; ++t, cc = wk.first_from(cc + 1)) {
                const int gi = gt + t;
                const bool fl_doc = wk.code(cc) == QC_DOC;
                const int kb0 = (lo + cc) * kBlk;
                const int kb1 = min(kb0 + kBlk, mk.N);
                const bool fl_bound = (kb0 + kBlk > mk.N) || (mk.causal && kb1 - 1 > q0 + mk.gap);
                const int k0 = kb0 + cbase;  // first key column of this thread
                const uint32_t tS = tmem + lane_base + uint32_t(gi & 1) * 128u + uint32_t(cbase);
                ok = mbar_wait(BAR(B_SFULL + (gi & 1)), (gi >> 1) & 1, ab, ST_WAIT_TIMEOUT + 27);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                uint32_t sr[64];
                tmem_ld32(tS, sr);
                tmem_ld32(tS + 32u, sr + 32);
                tc_wait_ld();
                float* pr = reinterpret_cast<float*>(sr);
                {
                    // P = exp2(S*c - LSE) on packed pairs
                    const uint64_t c2 = pack_f2(c, c), nl2 = pack_f2(-lse, -lse);
#pragma unroll
                    for (int x = 0; x < 32; ++x) {
                        float x0, x1;
                        unpack_f2(fma_f2(pack_f2(pr[2 * x], pr[2 * x + 1]), c2, nl2), x0, x1);
                        pr[2 * x] = fast_exp2(x0);
                        pr[2 * x + 1] = fast_exp2(x1);
                    }
                }
                if (fl_bound || fl_doc) {
                    int lim = 63;
                    if (fl_bound) {
                        int jmax = mk.N - 1;
                        if (mk.causal) jmax = min(jmax, row + mk.gap);
                        lim = jmax - k0;
                    }
                    if (fl_doc && qc < 0) {
                        const int4* kc4 = reinterpret_cast<const int4*>(mk.plan + mk.L.off_kc + bh_ids * mk.L.Npad + k0);
#pragma unroll
                        for (int q = 0; q < 16; ++q) {
                            const int4 kc = __ldg(kc4 + q);
                            pr[4 * q + 0] = (kc.x == qc && 4 * q + 0 <= lim) ? pr[4 * q + 0] : 0.f;
                            pr[4 * q + 1] = (kc.y == qc && 4 * q + 1 <= lim) ? pr[4 * q + 1] : 0.f;
                            pr[4 * q + 2] = (kc.z == qc && 4 * q + 2 <= lim) ? pr[4 * q + 2] : 0.f;
                            pr[4 * q + 3] = (kc.w == qc && 4 * q + 3 <= lim) ? pr[4 * q + 3] : 0.f;
                        }
                    } else {
#pragma unroll
                        for (int x = 0; x < 64; ++x) pr[x] = (x <= lim) ? pr[x] : 0.f;
                    }
                }
                ok = mbar_wait(BAR(B_DPFULL), gi & 1, ab, ST_WAIT_TIMEOUT + 28);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                uint32_t pk[32];
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    uint32_t dp[32];
                    tmem_ld32(tmem + lane_base + 256u + uint32_t(cbase) + uint32_t(q) * 32u, dp);
                    tc_wait_ld();
                    // masked entries have P == 0 exactly and dP - delta is finite, so dS is 0 there
                    // (flash_triton.py:400-414)
                    const uint64_t nd2 = pack_f2(-delta, -delta);
#pragma unroll
                    for (int x = 0; x < 16; ++x) {
                        float d0, d1;
                        unpack_f2(mul_f2(pack_f2(pr[32 * q + 2 * x], pr[32 * q + 2 * x + 1]),
                                         add_f2(pack_f2(__uint_as_float(dp[2 * x]), __uint_as_float(dp[2 * x + 1])), nd2)),
                                  d0, d1);
                        pk[16 * q + x] = pack2<BF16>(d0, d1);
                    }
                }
                tmem_st32(tS, pk);
                tc_wait_st();
                tc_fence_before();
                mbar_arrive(BAR(B_DSFULL + (gi & 1)));
            }
            if (!ok) break;

            // ------------------------------ item epilogue ------------------------------
            if (T > 0) {
                ok = mbar_wait(BAR(B_DONE), kk & 1, ab, ST_WAIT_TIMEOUT + 29);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
            }
            tc_fence_after();
            {
                // dQ * sm_scale (flash_triton.py:425) goes out through shared memory: each thread writes
                // its half row into the item's (now dead) Q tile in the tensor map's 128-byte-swizzled
                // layout; the producer warp issues the TMA store, which clips rows >= M.
                constexpr int HALF = D / 2;
                const uint32_t c0 = uint32_t(w) * HALF;
                uint8_t* stage = smem + S::off_q + s * S::TILE;
#pragma unroll
                for (int q = 0; q < HALF / 32; ++q) {
                    uint32_t x[32];
                    // tcgen05.ld is warp-collective: always executed, the values are ignored for an item without tiles
                    tmem_ld32(tmem + lane_base + 384u + c0 + uint32_t(q) * 32u, x);
                    tc_wait_ld();
                    uint32_t out[16];
#pragma unroll
                    for (int y = 0; y < 16; ++y) {
                        const float v0 = (T > 0) ? __uint_as_float(x[2 * y]) * p.sm_scale : 0.f;
                        const float v1 = (T > 0) ? __uint_as_float(x[2 * y + 1]) * p.sm_scale : 0.f;
                        out[y] = pack2<BF16>(v0, v1);
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int cg = int(c0) / 8 + 4 * q + i;  // 16-byte chunk of the row
                        const int box = cg >> 3, ch = cg & 7;
                        uint4* dst = reinterpret_cast<uint4*>(stage + box * S::BOX + r * 128 + ((ch ^ (r & 7)) << 4));
                        *dst = make_uint4(out[4 * i], out[4 * i + 1], out[4 * i + 2], out[4 * i + 3]);
                    }
                }
            }
            // the accumulator has been read: warp 9 may start the next item's dQ
            tc_fence_before();
            if (T > 0) {
                mbar_arrive(BAR(B_ACCFREE));
                ++kk;
            }
            fence_proxy_async();
            mbar_arrive(BAR(B_STAGED + s));  // the producer warp issues the TMA store
            gt += T;
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR(B_ITEMEMPTY + s));
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

template <int D, bool BF16>
static cudaError_t launch_dq_t(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                               const CUtensorMap& tdo, const CUtensorMap& tdq, const DqParams& p, int num_sms,
                               cudaStream_t stream) {
    auto kern = bwd_dq_kernel<D, BF16>;
    constexpr int smem = DqSmem<D>::total;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    const int n_items = p.mask.L.nQ * p.H * p.B;
    const int grid = n_items < num_sms ? n_items : num_sms;
    kern<<<grid, kAttnThreads, smem, stream>>>(tq, tk, tv, tdo, tdq, p);
    return cudaGetLastError();
}


cudaError_t launch_bwd_dq(int D, bool bf16, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                          const CUtensorMap& tdo, const CUtensorMap& tdq, const DqParams& p, int num_sms, cudaStream_t stream) {
    if (D == 128) return bf16 ? launch_dq_t<128, true>(tq, tk, tv, tdo, tdq, p, num_sms, stream)
                              : launch_dq_t<128, false>(tq, tk, tv, tdo, tdq, p, num_sms, stream);
    return bf16 ? launch_dq_t<64, true>(tq, tk, tv, tdo, tdq, p, num_sms, stream)
                : launch_dq_t<64, false>(tq, tk, tv, tdo, tdq, p, num_sms, stream);
}

}  // namespace fa
