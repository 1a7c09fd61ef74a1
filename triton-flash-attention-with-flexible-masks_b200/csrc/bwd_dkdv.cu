// dK / dV kernel. Replaces `_bwd_kv_kernel` (flash_triton.py:175-321) and the grouped-query
// sum that follows it (:635-637): per block of 128 keys, walk the visited query tiles of every
// query head of the group, recompute P, and accumulate dV += P^T dO, dK += dS^T Q in fp32.
//
// The tile is kept transposed (rows = keys, columns = queries): S^T = K Q^T and dP^T = V dO^T
// land in TMEM with one key per lane. P^T (input dtype) is written to a shared-memory tile in the
// K-major swizzled layout and is the A operand of dV += P^T dO; because it does not live in the
// S^T columns, S^T of the next tile is issued as soon as the scores have been read into
// registers and overlaps the whole exp / mask phase. dS^T goes back to TMEM over dP^T and is the
// A operand of dK += dS^T Q. dO and Q are read as MN-major B operands from their TMA tiles.
//
// Persistent: min(items, SMs) CTAs, item = one key block of one (batch, kv head), taken round
// robin. 12 warps:
//   warps 0-7  two compute groups; thread r of group g owns key row r and query columns
//              [64g, 64g+64) of every tile
//   warp 8     TMA producer (K, V per item; Q ring with the per-row LSE / delta; dO ring) and the
//              TMA stores of the finished item's dK / dV
//   warp 9     tcgen05.mma issuer for S^T; owns the TMEM allocation
//   warp 10    tcgen05.mma issuer for dV, dK and dP^T
//   warp 11    scheduler: per item, the range of candidate query blocks and their flags
// The Q / dO rings and all per-tile barriers run across item boundaries, so the next item's K and
// V and first Q / dO tiles are in flight and its first S^T is computed while the compute groups drain
// the accumulators of the finished item (dK and dV are staged in the Q and dO ring stage of the
// item's last tile, which is dead by then; that stage is refilled when the stores have read it).
// TMEM columns: S^T [0,128)  dP^T [128,256)  dV [256,256+D)  dK [256+D,256+2D).
#include "common.cuh"
#include "params.cuh"

namespace fa {

template <int D>
struct DkdvSmem {
    static constexpr int NST = (D == 128) ? 2 : 3;
    static constexpr int TILE = kBlk * D * 2;
    static constexpr int BOX = kBlk * 64 * 2;
    static constexpr int NBOX = D / 64;
    static constexpr int PT = kBlk * kBlk * 2;  // P^T tile: 128 keys x 128 queries
    static constexpr int VEC = 2 * kBlk * 4;    // lse, delta of one query block
    static constexpr int FLAGS = kListCap / 4;  // one item's candidate flags, 2 bits each
    static constexpr int off_k = 0;
    static constexpr int off_v = TILE;
    static constexpr int off_q = 2 * TILE;
    static constexpr int off_do = off_q + NST * TILE;
    static constexpr int off_p = off_do + NST * TILE;
    static constexpr int off_vec = off_p + PT;
    static constexpr int off_flags = off_vec + NST * VEC;  // two item slots
    static constexpr int off_info = off_flags + 2 * FLAGS;  // two item slots x {lo, n, tiles, item, key block, kv head, batch, -}
    static constexpr int off_bar = off_info + 64;
    // k_full, v_full, k_empty, q_full[NST], do_full[NST], q_empty[NST], do_empty[NST], s_full, s_free,
    // dp_full, p_full, p_free, ds_full, done, acc_free, staged, stage_free, item_full[2], item_empty[2], v_empty
    static constexpr int n_bar = 3 + 4 * NST + 10 + 4 + 1;
    static constexpr int off_misc = off_bar + n_bar * 8;
    static constexpr int total = off_misc + 16;
};
static_assert(DkdvSmem<128>::total <= 232448 && DkdvSmem<64>::total <= 232448, "shared memory budget");

// Per-candidate code kept in shared memory (2 bits): 0 not visited, 1 visited without id check,
// 2 id check, 3 id check and the query codes of the block are monotone. Whether a tile needs the
// range check (causal bound and / or query tail) follows from its coordinates alone.
enum : uint32_t { KC_SKIP = 0u, KC_PLAIN = 1u, KC_DOC = 2u, KC_DOCMONO = 3u };

// Flags of tile (qb, kb) for all query heads of one kv head at once. When the heads disagree
// (ids given per head) the id check is forced, entry by entry, which is always exact.
__device__ __forceinline__ uint32_t classify_group(const MaskArgs& mk, int b, int hk, int G, int qb, int kb) {
    if (mk.He == 1 || G == 1) return classify_from_plan(mk, b, mk.He == 1 ? 0 : hk * G, qb, kb);
    uint32_t f = 0, mono = TILE_KMONO | TILE_QMONO;
    bool all = true;
    for (int g = 0; g < G; ++g) {
        const uint32_t fg = classify_from_plan(mk, b, hk * G + g, qb, kb);
        if (fg & TILE_VISIT) { f |= fg; mono &= fg; } else all = false;
    }
    // the chunk shortcuts of the id check may only be taken if the codes are monotone for every head
    // that the check is applied to (a head that reports no id check does not report its monotony)
    f &= ~(TILE_KMONO | TILE_QMONO);
    if (f && !all) f |= TILE_DOC;
    else f |= mono;
    return f;
}

// Walks the visited candidates of an item for all heads of the group, head-major:
// (g, c) -> next visited candidate; c == n means "past the end".
struct Walk {
    const uint8_t* fl;
    int n;
    __device__ __forceinline__ uint32_t code(int c) const { return (uint32_t(fl[c >> 2]) >> (2 * (c & 3))) & 3u; }
    __device__ __forceinline__ int first_from(int c) const {
        while (c < n && code(c) == KC_SKIP) ++c;
        return c;
    }
    __device__ __forceinline__ void advance(int& g, int& c) const {
        c = first_from(c + 1);
        if (c >= n) { g += 1; c = first_from(0); }
    }
};

template <int D, bool BF16>
__global__ void __launch_bounds__(kAttnThreads, 1)
bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                const __grid_constant__ CUtensorMap tmdK, const __grid_constant__ CUtensorMap tmdV,
                const DkdvParams p) {
    using S = DkdvSmem<D>;
    constexpr int NST = S::NST;
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const MaskArgs& mk = p.mask;
    const int G = p.G;
    const int nK = mk.L.nK;
    const int n_items = nK * p.Hk * p.B;
    unsigned int* ctr = mk.ctr ? mk.ctr + CTR_DKDV : nullptr;
    // item -> (key block, kv head, batch). Heads are taken in groups of p.gh; inside a group the key
    // blocks go in order (with a causal mask: long ones first) and the heads of the group vary
    // fastest. The CTAs thus work on neighbouring key blocks of a few heads at a time: few enough
    // that their Q / dO streams stay in L2, enough that not all CTAs pull the same lines.
    const int HB = p.Hk * p.B;
    auto decode = [&](int j, int& kb, int& hk, int& b) {
        const int per = p.gh * nK;
        const int grp = j / per, rem = j - grp * per;
        const int gsz = min(p.gh, HB - grp * p.gh);
        const int pos = rem / gsz, bh = grp * p.gh + (rem - pos * gsz);
        hk = bh % p.Hk;
        b = bh / p.Hk;
        // few items per CTA: longest first (sorted in the plan), so that no long item is left for the end
        kb = p.by_length ? mk.plan[mk.L.off_ordk + (int64_t(b) * mk.He + (mk.He == 1 ? 0 : hk * G)) * nK + pos] : pos;
    };

    volatile int* misc = reinterpret_cast<volatile int*>(smem + S::off_misc);
    volatile int* info = reinterpret_cast<volatile int*>(smem + S::off_info);
    const uint32_t bar0 = sbase + S::off_bar;
    auto BAR = [&](int i) { return bar0 + 8u * uint32_t(i); };
    const int B_KFULL = 0, B_VFULL = 1, B_KEMPTY = 2, B_QFULL = 3, B_DOFULL = B_QFULL + NST, B_QEMPTY = B_DOFULL + NST,
              B_DOEMPTY = B_QEMPTY + NST, B_SFULL = B_DOEMPTY + NST, B_SFREE = B_SFULL + 1, B_DPFULL = B_SFULL + 2,
              B_PFULL = B_SFULL + 3, B_PFREE = B_SFULL + 4, B_DSFULL = B_SFULL + 5, B_DONE = B_SFULL + 6,
              B_ACCFREE = B_SFULL + 7, B_STAGED = B_SFULL + 8, B_STAGEFREE = B_SFULL + 9, B_ITEMFULL = B_SFULL + 10,
              B_ITEMEMPTY = B_ITEMFULL + 2, B_VEMPTY = B_ITEMEMPTY + 2;
    Abort ab{misc + 1, p.status, p.wait_limit};

    const uint32_t sK = sbase + S::off_k, sV = sbase + S::off_v, sP = sbase + S::off_p;
    auto sQ = [&](int s) { return sbase + S::off_q + uint32_t(s) * S::TILE; };
    auto sdO = [&](int s) { return sbase + S::off_do + uint32_t(s) * S::TILE; };
    auto sVec = [&](int s) { return sbase + S::off_vec + uint32_t(s) * S::VEC; };
    auto walk_of = [&](int s, int n) { return Walk{smem + S::off_flags + s * S::FLAGS, n}; };

    if (tid == 0) {
        mbar_init(BAR(B_KFULL), 1); mbar_init(BAR(B_VFULL), 1); mbar_init(BAR(B_KEMPTY), 1);
        for (int s = 0; s < NST; ++s) {
            mbar_init(BAR(B_QFULL + s), 1); mbar_init(BAR(B_DOFULL + s), 1);
            mbar_init(BAR(B_QEMPTY + s), 2);  // S^T (warp 9) and dK (warp 10) both read the Q stage
            mbar_init(BAR(B_DOEMPTY + s), 1); // dP^T and dV are issued by the same thread: one commit
        }
        mbar_init(BAR(B_SFULL), 1);
        mbar_init(BAR(B_SFREE), 256);
        mbar_init(BAR(B_DPFULL), 1);
        mbar_init(BAR(B_PFULL), 256);
        mbar_init(BAR(B_PFREE), 1);
        mbar_init(BAR(B_DSFULL), 256);
        mbar_init(BAR(B_DONE), 1);  // warp 10 only: warp 9 runs ahead into the next item
        mbar_init(BAR(B_ACCFREE), 256);
        mbar_init(BAR(B_STAGED), 256);
        mbar_init(BAR(B_STAGEFREE), 1);
        mbar_init(BAR(B_VEMPTY), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(BAR(B_ITEMFULL + s), 1);
            mbar_init(BAR(B_ITEMEMPTY + s), 11);  // producer, two MMA issuers, eight compute warps
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
    if (aborted && (sbase & 1023u) == 0) nan_fill_outputs(smem + S::off_k, S::NBOX, &tmdK, &tmdV, nK, p.Hk, p.B);

    if (warp >= 8) {
        setmaxnreg_dec<56>();
        if (aborted) {
        } else if (warp == 11) {
            // ------------------------------ scheduler ------------------------------
            // Item k goes to slot k & 1: range [lo, lo + n) of candidate query blocks (union over the
            // group's heads), a 2-bit code per candidate, and the number of tiles.
            // Items are handed out in order from a counter in the plan (any CTA takes the next one: the
            // work per item varies with the mask); without counters (no plan given) they are
            // dealt out round robin in alternating direction, which evens out their sorted lengths.
            bool ok = true;
            for (int k = 0;; ++k) {
                const int s = k & 1, use = k >> 1;
                if (use > 0) ok = mbar_wait(BAR(B_ITEMEMPTY + s), (use - 1) & 1, ab, ST_WAIT_TIMEOUT + 54);
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
                        info[s * 8 + 3] = -1;
                        mbar_arrive(BAR(B_ITEMFULL + s));
                    }
                    break;
                }
                int kb, hk, b;
                decode(j, kb, hk, b);
                int lo = 0x7fffffff, hi = 0;
                {
                    const int ng = (mk.He == 1) ? 1 : G;
                    for (int g = 0; g < ng; ++g) {
                        int l, h2;
                        q_range(mk, b, mk.He == 1 ? 0 : hk * G + g, kb, l, h2);
                        if (h2 > l) { lo = min(lo, l); hi = max(hi, h2); }
                    }
                    if (hi == 0) lo = 0;
                }
                int n = hi - lo;
                if (n > kListCap) n = kListCap;
                uint8_t* fl = smem + S::off_flags + s * S::FLAGS;
                int cnt = 0;
                for (int i = lane; 4 * i < n; i += 32) {
                    uint32_t byte = 0;
                    for (int e = 0; e < 4; ++e) {
                        const int c = 4 * i + e;
                        if (c >= n) break;
                        const uint32_t f = classify_group(mk, b, hk, G, lo + c, kb);
                        uint32_t code = KC_SKIP;
                        if (f & TILE_VISIT) code = !(f & TILE_DOC) ? KC_PLAIN : (f & TILE_QMONO) ? KC_DOCMONO : KC_DOC;
                        cnt += (code != KC_SKIP);
                        byte |= code << (2 * e);
                    }
                    fl[i] = uint8_t(byte);
                }
                for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
                __syncwarp();
                if (lane == 0) {
                    info[s * 8 + 0] = lo;
                    info[s * 8 + 1] = n;
                    info[s * 8 + 2] = cnt * G;  // tiles of all query heads of the group, head-major
                    info[s * 8 + 3] = j;
                    info[s * 8 + 4] = kb;
                    info[s * 8 + 5] = hk;
                    info[s * 8 + 6] = b;
                    mbar_arrive(BAR(B_ITEMFULL + s));
                }
            }
        } else if (warp == 8) {
            // ------------------------------ TMA producer ------------------------------
            if (lane == 0) {
                tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmdO); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
                tma_prefetch_desc(&tmdK); tma_prefetch_desc(&tmdV);
                bool ok = true;
                int k = 0, kk = 0;  // items, items with tiles
                int gt = 0;         // tiles of all earlier items (stage / phase of the Q and dO rings)
                int pkb = 0, phk = 0, pb = 0;  // the previous item, whose dK / dV are still to be stored
                // stores the dV / dK of item i, staged in the dO / Q ring stage `st`, and frees the stage
                auto finish_store = [&](int i, int kb, int hk, int b, int st) {
                    bool o = mbar_wait(BAR(B_STAGED), i & 1, ab, ST_WAIT_TIMEOUT + 55);
                    if (!o) return false;
                    if (misc[1] == 0) {
                        for (int x = 0; x < S::NBOX; ++x) {
                            tma_store_4d(&tmdV, sdO(st) + x * S::BOX, x * 64, kb * kBlk, hk, b);
                            tma_store_4d(&tmdK, sQ(st) + x * S::BOX, x * 64, kb * kBlk, hk, b);
                        }
                        tma_store_commit();
                        tma_store_wait_read();
                    }
                    mbar_arrive(BAR(B_STAGEFREE));
                    return true;
                };
                for (;; ++k) {
                    const int s = k & 1;
                    ok = mbar_wait(BAR(B_ITEMFULL + s), (k >> 1) & 1, ab, ST_WAIT_TIMEOUT + 56);
                    if (!ok) break;
                    const int lo = info[s * 8 + 0], n = info[s * 8 + 1], NIT = info[s * 8 + 2], j = info[s * 8 + 3];
                    if (j < 0) break;
                    const int kb = info[s * 8 + 4], hk = info[s * 8 + 5], b = info[s * 8 + 6];
                    const Walk wk = walk_of(s, n);
                    int cg = 0, cc = wk.first_from(0);
                    auto load_qdo = [&](int it) {
                        const int h = hk * G + cg;
                        const int qb = lo + cc;
                        const int gi = gt + it, st = gi % NST, use = gi / NST;
                        if (use > 0 && !mbar_wait(BAR(B_QEMPTY + st), (use - 1) & 1, ab, ST_WAIT_TIMEOUT + 41)) return false;
                        mbar_expect_tx(BAR(B_QFULL + st), S::TILE + S::VEC);
                        for (int x = 0; x < S::NBOX; ++x)
                            tma_load_4d(sQ(st) + x * S::BOX, &tmQ, BAR(B_QFULL + st), x * 64, qb * kBlk, h, b);
                        const int64_t roff = (int64_t(b) * p.H + h) * mk.L.Mpad + int64_t(qb) * kBlk;
                        bulk_load_1d(sVec(st), p.lse + roff, kBlk * 4, BAR(B_QFULL + st));
                        bulk_load_1d(sVec(st) + kBlk * 4, p.delta + roff, kBlk * 4, BAR(B_QFULL + st));
                        if (use > 0 && !mbar_wait(BAR(B_DOEMPTY + st), (use - 1) & 1, ab, ST_WAIT_TIMEOUT + 42)) return false;
                        mbar_expect_tx(BAR(B_DOFULL + st), S::TILE);
                        for (int x = 0; x < S::NBOX; ++x)
                            tma_load_4d(sdO(st) + x * S::BOX, &tmdO, BAR(B_DOFULL + st), x * 64, qb * kBlk, h, b);
                        wk.advance(cg, cc);
                        return true;
                    };
                    // The previous item is staged in ring stage (gt + NST - 1) % NST, the stage of its last
                    // tile. K, V and the tiles of the other stages do not wait for its epilogue.
                    const int npre = NIT < NST - 1 ? NIT : NST - 1;
                    if (NIT > 0) {
                        if (kk > 0) ok = mbar_wait(BAR(B_KEMPTY), (kk - 1) & 1, ab, ST_WAIT_TIMEOUT + 57);
                        if (!ok) break;
                        mbar_expect_tx(BAR(B_KFULL), S::TILE);
                        for (int x = 0; x < S::NBOX; ++x) tma_load_4d(sK + x * S::BOX, &tmK, BAR(B_KFULL), x * 64, kb * kBlk, hk, b);
                        if (kk > 0) ok = mbar_wait(BAR(B_VEMPTY), (kk - 1) & 1, ab, ST_WAIT_TIMEOUT + 60);
                        if (!ok) break;
                        mbar_expect_tx(BAR(B_VFULL), S::TILE);
                        for (int x = 0; x < S::NBOX; ++x) tma_load_4d(sV + x * S::BOX, &tmV, BAR(B_VFULL), x * 64, kb * kBlk, hk, b);
                        for (int it = 0; it < npre && ok; ++it) ok = load_qdo(it);
                        if (!ok) break;
                    }
                    if (k > 0) ok = finish_store(k - 1, pkb, phk, pb, (gt + NST - 1) % NST);
                    if (!ok) break;
                    if (NIT > 0) {
                        for (int it = npre; it < NIT && ok; ++it) ok = load_qdo(it);
                        if (!ok) break;
                        ++kk;
                    }
                    gt += NIT;
                    pkb = kb; phk = hk; pb = b;
                    mbar_arrive(BAR(B_ITEMEMPTY + s));
                }
                if (ok && k > 0) finish_store(k - 1, pkb, phk, pb, (gt + NST - 1) % NST);
            }
        } else {
            // ------------------------------ MMA issuers (warps 9, 10) ------------------------------
            //   warp 9 : S^T(it) = K Q^T, as soon as the compute groups have read S^T(it-1)
            //   warp 10: dV(it) += P^T dO when P^T is in shared memory, then dK(it) += dS^T Q and
            //            dP^T(it+1) = V dO^T when dS^T is in TMEM (dP^T overwrites dS^T: same thread)
            // Each Q / dO stage is read by both threads, so its "empty" barrier takes two commits.
            if (lane == 0) {
                constexpr uint32_t idesc_s = make_idesc(BF16, 128, 128, false, false);
                constexpr uint32_t idesc_d = make_idesc(BF16, 128, D, false, true);
                constexpr uint64_t desc_mn = desc_mn_major(S::BOX);
                auto q_ready = [&](int gi) { return mbar_wait(BAR(B_QFULL + gi % NST), (gi / NST) & 1, ab, ST_WAIT_TIMEOUT + 44); };
                auto do_ready = [&](int gi) { return mbar_wait(BAR(B_DOFULL + gi % NST), (gi / NST) & 1, ab, ST_WAIT_TIMEOUT + 45); };
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
                    ok = mbar_wait(BAR(B_ITEMFULL + s), (k >> 1) & 1, ab, ST_WAIT_TIMEOUT + 56);
                    if (!ok) break;
                    const int NIT = info[s * 8 + 2];
                    if (info[s * 8 + 3] < 0) break;
                    if (NIT > 0 && warp == 9) {
                        ok = mbar_wait(BAR(B_KFULL), kk & 1, ab, ST_WAIT_TIMEOUT + 43);
                        for (int it = 0; it < NIT && ok; ++it) {
                            const int gi = gt + it, st = gi % NST;
                            ok = q_ready(gi);
                            // the S^T columns are free once every compute thread has loaded the previous S^T
                            if (ok && gi > 0) ok = mbar_wait(BAR(B_SFREE), (gi - 1) & 1, ab, ST_WAIT_TIMEOUT + 46);
                            if (!ok) break;
                            tc_fence_after();
                            ss_mmas(tmem, sK, sQ(st));
                            umma_commit(BAR(B_QEMPTY + st));
                            umma_commit(BAR(B_SFULL));
                        }
                        if (!ok) break;
                        umma_commit(BAR(B_KEMPTY));
                    } else if (NIT > 0) {
                        ok = mbar_wait(BAR(B_VFULL), kk & 1, ab, ST_WAIT_TIMEOUT + 43);
                        if (ok) ok = do_ready(gt);
                        if (!ok) break;
                        tc_fence_after();
                        ss_mmas(tmem + 128u, sV, sdO(gt % NST));  // dP^T(0)
                        umma_commit(BAR(B_DPFULL));
                        if (NIT == 1) umma_commit(BAR(B_VEMPTY));  // V may be replaced after the item's last dP^T
                        // dV(0) and dK(0) overwrite the accumulators: the previous item's epilogue must have read them
                        if (kk > 0) ok = mbar_wait(BAR(B_ACCFREE), (kk - 1) & 1, ab, ST_WAIT_TIMEOUT + 58);
                        for (int it = 0; it < NIT && ok; ++it) {
                            const int gi = gt + it, st = gi % NST;
                            const bool more = it + 1 < NIT;
                            // dV(it) += P^T dO: A = P^T from shared memory (K-major), B = dO (MN-major)
                            ok = mbar_wait(BAR(B_PFULL), gi & 1, ab, ST_WAIT_TIMEOUT + 47);
                            if (!ok) break;
                            tc_fence_after();
#pragma unroll
                            for (int kk2 = 0; kk2 < kBlk / 16; ++kk2) {
                                const uint32_t off = uint32_t(kk2 >> 2) * S::BOX + uint32_t(kk2 & 3) * 32u;
                                umma_ss(tmem + 256u, smem_desc_at(kDescKMajor, sP + off),
                                        smem_desc_at(desc_mn, sdO(st) + uint32_t(kk2) * 2048u), idesc_d, (it > 0 || kk2 > 0) ? 1u : 0u);
                            }
                            umma_commit(BAR(B_PFREE));
                            umma_commit(BAR(B_DOEMPTY + st));
                            if (more) ok = do_ready(gi + 1);
                            if (ok) ok = mbar_wait(BAR(B_DSFULL), gi & 1, ab, ST_WAIT_TIMEOUT + 48);
                            if (!ok) break;
                            tc_fence_after();
                            // dK(it) += dS^T Q: A = dS^T from TMEM, B = Q (MN-major)
#pragma unroll
                            for (int kk2 = 0; kk2 < kBlk / 16; ++kk2) {
                                const uint32_t acol = (kk2 < 4) ? uint32_t(kk2) * 8u : 64u + uint32_t(kk2 - 4) * 8u;
                                umma_ts(tmem + 256u + uint32_t(D), tmem + 128u + acol,
                                        smem_desc_at(desc_mn, sQ(st) + uint32_t(kk2) * 2048u), idesc_d, (it > 0 || kk2 > 0) ? 1u : 0u);
                            }
                            umma_commit(BAR(B_QEMPTY + st));
                            if (more) {
                                ss_mmas(tmem + 128u, sV, sdO((gi + 1) % NST));  // dP^T(it+1)
                                umma_commit(BAR(B_DPFULL));
                                if (it + 2 == NIT) umma_commit(BAR(B_VEMPTY));
                            }
                        }
                        if (!ok) break;
                        umma_commit(BAR(B_DONE));
                    }
                    if (NIT > 0) ++kk;
                    gt += NIT;
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
        const int cbase = 64 * w;  // first query column of this thread inside a tile
        const float c = p.scale_log2;
        bool ok = !aborted;
        const uint32_t tS = tmem + lane_base + uint32_t(cbase);
        const uint32_t tdP = tmem + lane_base + 128u + uint32_t(cbase);
        int k = 0, kk = 0, gt = 0;
        for (; ok; ++k) {
            const int s = k & 1;
            ok = mbar_wait(BAR(B_ITEMFULL + s), (k >> 1) & 1, ab, ST_WAIT_TIMEOUT + 56);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const int lo = info[s * 8 + 0], n = info[s * 8 + 1], NIT = info[s * 8 + 2], jt = info[s * 8 + 3];
            if (jt < 0) break;
            const int kb = info[s * 8 + 4], hk = info[s * 8 + 5], b = info[s * 8 + 6];
            const Walk wk = walk_of(s, n);
            const int j = kb * kBlk + r;  // this thread's key
            const int k0 = kb * kBlk, k1 = min(k0 + kBlk, mk.N);

            int cg = 0, cc = wk.first_from(0);
            int kc = 0, kc_g = -1;  // this key's code for the current query head
            for (int it = 0; it < NIT && ok; ++it, wk.advance(cg, cc)) {
                const int he = (mk.He == 1) ? 0 : hk * G + cg;
                const uint32_t code = wk.code(cc);
                const bool fl_doc = code >= KC_DOC;
                const int qb0 = (lo + cc) * kBlk;
                const bool fl_range = (mk.causal && (k0 + kBlk > mk.N || k1 - 1 > qb0 + mk.gap)) || (qb0 + kBlk > mk.M);
                const int q0 = qb0 + cbase;  // first query row of this thread's columns
                const int gi = gt + it, st = gi % NST;
                const float* vlse = reinterpret_cast<const float*>(smem + S::off_vec + st * S::VEC) + cbase;
                const float* vdelta = vlse + kBlk;

                ok = mbar_wait(BAR(B_QFULL + st), (gi / NST) & 1, ab, ST_WAIT_TIMEOUT + 49);
                if (ok) ok = mbar_wait(BAR(B_SFULL), gi & 1, ab, ST_WAIT_TIMEOUT + 50);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                uint32_t sr[64];
                tmem_ld32(tS, sr);
                tmem_ld32(tS + 32u, sr + 32);
                tc_wait_ld();
                tc_fence_before();
                mbar_arrive(BAR(B_SFREE));  // the next S^T may now overwrite the columns
                float* pr = reinterpret_cast<float*>(sr);
                {
                    // P^T = exp2(S^T*c - LSE) on packed pairs. A fully masked row has LSE = -inf and only
                    // occurs in flagged tiles.
                    const uint64_t c2 = pack_f2(c, c);
#pragma unroll
                    for (int q = 0; q < 16; ++q) {
                        const float4 l4 = *reinterpret_cast<const float4*>(vlse + 4 * q);
                        float x0, x1, x2, x3;
                        unpack_f2(fma_f2(pack_f2(pr[4 * q + 0], pr[4 * q + 1]), c2, pack_f2(-l4.x, -l4.y)), x0, x1);
                        unpack_f2(fma_f2(pack_f2(pr[4 * q + 2], pr[4 * q + 3]), c2, pack_f2(-l4.z, -l4.w)), x2, x3);
                        pr[4 * q + 0] = fast_exp2(x0);
                        pr[4 * q + 1] = fast_exp2(x1);
                        pr[4 * q + 2] = fast_exp2(x2);
                        pr[4 * q + 3] = fast_exp2(x3);
                    }
                }
                if (fl_range || fl_doc) {
                    // keep(x) = (cmin <= x < cmax) & (qc[x] >= 0 | qc[x] == kc), per 32-query chunk where
                    // the chunk lies on one side of the range and (monotone query codes) is one document
                    int cmin = -0x40000000, cmax = 64;
                    if (fl_range) {
                        if (mk.causal) cmin = (j - mk.gap) - q0;
                        cmax = min(64, mk.M - q0);
                    }
                    const int* qcs = nullptr;
                    if (fl_doc) {
                        const int64_t bh_ids = int64_t(b) * mk.He + he;
                        if (kc_g != cg) { kc = mk.plan[mk.L.off_kc + bh_ids * mk.L.Npad + j]; kc_g = cg; }
                        qcs = mk.plan + mk.L.off_qc + bh_ids * mk.L.Mpad + q0;
                    }
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        int state = 0;  // this key in chunk q: 0 keep all, 1 mask all, 2 entry by entry
                        if (32 * q >= cmax || 32 * q + 31 < cmin) state = 1;
                        else if (32 * q < cmin || 32 * q + 31 >= cmax) state = 2;
                        if (fl_doc && state != 1) {
                            if (code == KC_DOCMONO) {
                                const int qf = __ldg(qcs + 32 * q), ql = __ldg(qcs + 32 * q + 31);
                                if (qf != ql) state = 2;
                                else if (!(qf >= 0 || qf == kc)) state = 1;
                            } else {
                                state = 2;
                            }
                        }
                        if (!__any_sync(0xffffffffu, state == 2)) {
                            if (state == 1) {
#pragma unroll
                                for (int x = 0; x < 32; ++x) pr[32 * q + x] = 0.f;
                            }
                        } else if (fl_doc) {
                            const int4* qc4 = reinterpret_cast<const int4*>(qcs + 32 * q);
#pragma unroll
                            for (int u = 0; u < 8; ++u) {
                                const int4 qc = __ldg(qc4 + u);
                                const int x = 32 * q + 4 * u;
                                pr[x + 0] = ((qc.x >= 0 || qc.x == kc) && x + 0 >= cmin && x + 0 < cmax) ? pr[x + 0] : 0.f;
                                pr[x + 1] = ((qc.y >= 0 || qc.y == kc) && x + 1 >= cmin && x + 1 < cmax) ? pr[x + 1] : 0.f;
                                pr[x + 2] = ((qc.z >= 0 || qc.z == kc) && x + 2 >= cmin && x + 2 < cmax) ? pr[x + 2] : 0.f;
                                pr[x + 3] = ((qc.w >= 0 || qc.w == kc) && x + 3 >= cmin && x + 3 < cmax) ? pr[x + 3] : 0.f;
                            }
                        } else {
#pragma unroll
                            for (int x = 0; x < 32; ++x) pr[32 * q + x] = (32 * q + x >= cmin && 32 * q + x < cmax) ? pr[32 * q + x] : 0.f;
                        }
                    }
                }
                // P^T (input dtype) -> shared memory, K-major 128-byte-swizzled rows: this thread's 64
                // queries are one 128-byte row of box `w`. The previous tile's dV MMAs must have read the tile.
                if (gi > 0) ok = mbar_wait(BAR(B_PFREE), (gi - 1) & 1, ab, ST_WAIT_TIMEOUT + 51);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                {
                    uint8_t* prow = smem + S::off_p + w * S::BOX + r * 128;
#pragma unroll
                    for (int ch = 0; ch < 8; ++ch) {
                        uint4 v4;
                        v4.x = pack2<BF16>(pr[8 * ch + 0], pr[8 * ch + 1]);
                        v4.y = pack2<BF16>(pr[8 * ch + 2], pr[8 * ch + 3]);
                        v4.z = pack2<BF16>(pr[8 * ch + 4], pr[8 * ch + 5]);
                        v4.w = pack2<BF16>(pr[8 * ch + 6], pr[8 * ch + 7]);
                        *reinterpret_cast<uint4*>(prow + ((ch ^ (r & 7)) << 4)) = v4;
                    }
                }
                fence_proxy_async();
                mbar_arrive(BAR(B_PFULL));

                ok = mbar_wait(BAR(B_DPFULL), gi & 1, ab, ST_WAIT_TIMEOUT + 52);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                uint32_t pk[32];
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    uint32_t dp[32];
                    tmem_ld32(tdP + uint32_t(q) * 32u, dp);
                    tc_wait_ld();
                    // masked entries have P == 0 exactly and dP - delta is finite, so dS is 0 there
#pragma unroll
                    for (int x = 0; x < 16; ++x) {
                        const float2 dl = *reinterpret_cast<const float2*>(vdelta + 32 * q + 2 * x);
                        float d0, d1;
                        unpack_f2(mul_f2(pack_f2(pr[32 * q + 2 * x], pr[32 * q + 2 * x + 1]),
                                         add_f2(pack_f2(__uint_as_float(dp[2 * x]), __uint_as_float(dp[2 * x + 1])),
                                                pack_f2(-dl.x, -dl.y))),
                                  d0, d1);
                        pk[16 * q + x] = pack2<BF16>(d0, d1);
                    }
                }
                tmem_st32(tdP, pk);
                tc_wait_st();
                tc_fence_before();
                mbar_arrive(BAR(B_DSFULL));
            }
            if (!ok) break;

            // ------------------------------ item epilogue ------------------------------
            // the previous item's stores have read their staging stage (it may be the same one)
            if (k > 0) ok = mbar_wait(BAR(B_STAGEFREE), (k - 1) & 1, ab, ST_WAIT_TIMEOUT + 59);
            // dV is final (and the last dO tile dead) when the last dV MMAs are complete: it is drained
            // while the last dK MMAs still run
            if (ok && NIT > 0) ok = mbar_wait(BAR(B_PFREE), (gt + NIT - 1) & 1, ab, ST_WAIT_TIMEOUT + 51);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            {
                // dV and dK * sm_scale (flash_triton.py:313) go out through shared memory: each thread
                // writes its half rows into the dO and Q ring stage of the item's last tile (dead: all MMAs
                // of the item are complete) in the tensor maps' 128-byte-swizzled layout; the producer warp
                // issues the TMA stores, which clip rows >= N.
                const int sst = (gt + NIT + NST - 1) % NST;
                constexpr int HALF = D / 2;
                const uint32_t c0 = uint32_t(w) * HALF;
#pragma unroll
                for (int which = 0; which < 2; ++which) {  // 0: dV, 1: dK
                    if (which == 1 && NIT > 0) {
                        ok = mbar_wait(BAR(B_DONE), kk & 1, ab, ST_WAIT_TIMEOUT + 51);
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok) break;
                        tc_fence_after();
                    }
                    const float mul = which ? p.sm_scale : 1.0f;
                    uint8_t* stage = smem + (which ? S::off_q : S::off_do) + sst * S::TILE;
#pragma unroll
                    for (int q = 0; q < HALF / 32; ++q) {
                        uint32_t x[32];
                        // tcgen05.ld is warp-collective: always executed, the values are ignored for an item without tiles
                        tmem_ld32(tmem + lane_base + 256u + uint32_t(which * D) + c0 + uint32_t(q) * 32u, x);
                        tc_wait_ld();
                        uint32_t o16[16];
#pragma unroll
                        for (int y = 0; y < 16; ++y) {
                            const float v0 = (NIT > 0) ? __uint_as_float(x[2 * y]) * mul : 0.f;
                            const float v1 = (NIT > 0) ? __uint_as_float(x[2 * y + 1]) * mul : 0.f;
                            o16[y] = pack2<BF16>(v0, v1);
                        }
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int cgk = int(c0) / 8 + 4 * q + i;  // 16-byte chunk of the row
                            const int box = cgk >> 3, ch = cgk & 7;
                            uint4* dst = reinterpret_cast<uint4*>(stage + box * S::BOX + r * 128 + ((ch ^ (r & 7)) << 4));
                            *dst = make_uint4(o16[4 * i], o16[4 * i + 1], o16[4 * i + 2], o16[4 * i + 3]);
                        }
                    }
                }
            }
            if (!ok) break;
            // both accumulators have been read: warp 10 may start the next item's dV / dK
            tc_fence_before();
            if (NIT > 0) {
                mbar_arrive(BAR(B_ACCFREE));
                ++kk;
            }
            fence_proxy_async();
            mbar_arrive(BAR(B_STAGED));  // the producer warp issues the TMA stores
            gt += NIT;
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
static cudaError_t launch_dkdv_t(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                                 const CUtensorMap& tdo, const CUtensorMap& tdk, const CUtensorMap& tdv,
                                 const DkdvParams& p, int num_sms, cudaStream_t stream) {
    auto kern = bwd_dkdv_kernel<D, BF16>;
    constexpr int smem = DkdvSmem<D>::total;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    const int n_items = p.mask.L.nK * p.Hk * p.B;
    const int grid = n_items < num_sms ? n_items : num_sms;
    kern<<<grid, kAttnThreads, smem, stream>>>(tq, tk, tv, tdo, tdk, tdv, p);
    return cudaGetLastError();
}


cudaError_t launch_bwd_dkdv(int D, bool bf16, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                            const CUtensorMap& tdo, const CUtensorMap& tdk, const CUtensorMap& tdv,
                            const DkdvParams& p, int num_sms, cudaStream_t stream) {
    if (D == 128) return bf16 ? launch_dkdv_t<128, true>(tq, tk, tv, tdo, tdk, tdv, p, num_sms, stream)
                              : launch_dkdv_t<128, false>(tq, tk, tv, tdo, tdk, tdv, p, num_sms, stream);
    return bf16 ? launch_dkdv_t<64, true>(tq, tk, tv, tdo, tdk, tdv, p, num_sms, stream)
                : launch_dkdv_t<64, false>(tq, tk, tv, tdo, tdk, tdv, p, num_sms, stream);
}

}  // namespace fa
