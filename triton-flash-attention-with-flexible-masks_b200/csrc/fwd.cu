// Forward kernel: O = softmax(mask(Q K^T * sm_scale)) V and the row log-sum-exp.
// Replaces `_fwd_kernel` (flash_triton.py:25-141). Same mathematics (base-2 online softmax,
// P rounded to the input dtype before P*V, fp32 accumulation), except that the scale is
// applied in fp32 to the fp32 scores instead of being folded into a rounded Q
// (flash_triton.py:88), and tiles the mask plan proves empty are not visited at all.
//
// One CTA = one block of 128 queries of one (batch, head). 12 warps:
//   warps 0-3  softmax group 0, warps 4-7 softmax group 1 (thread r of a group owns row r)
//   warp 8     TMA producer (Q once, then K and V rings)
//   warps 9,10 tcgen05.mma issuers, one per softmax group; warp 9 owns the TMEM allocation
//   warp 11    idle; it only completes the third warpgroup so that registers can be moved
//              from it to the softmax groups (setmaxnreg works on whole warpgroups)
// Visited key tiles alternate between the two groups: tile t uses score buffer S[t&1] and
// accumulates into O[t&1] with its own running max / sum, so the tensor pipe computes
// S(t+1) while group t&1 is busy with the softmax of tile t. The two partial results are
// merged in the epilogue.  TMEM columns: S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [256+D, 256+2D).
// P (input dtype, two values per column) overwrites the first 64 columns of its S buffer.
#include <type_traits>
#include "common.cuh"
#include "params.cuh"
#include "trace.cuh"

namespace fa {

constexpr int kPolyOf4 = 1;  // of every 4 pairs of scores, how many take the FMA-pipe exp2

template <int D>
struct FwdSmem {
    static constexpr int NS = (D == 128) ? 3 : 4;
    static constexpr int TILE = kBlk * D * 2;
    static constexpr int BOX = kBlk * 64 * 2;
    static constexpr int NBOX = D / 64;
    static constexpr int off_q = 0;
    static constexpr int off_k = TILE;
    static constexpr int off_v = off_k + NS * TILE;
    static constexpr int off_list = off_v + NS * TILE;  // uint16 [kListCap]
    static constexpr int off_bar = off_list + kListCap * 2;
    // barriers (8 bytes each): q_full, k_full[NS], v_full[NS], k_empty[NS], v_empty[NS],
    // s_full[2], p_half0[2], p_half1[2], pv_done[2], turn[2]
    static constexpr int n_bar = 1 + 4 * NS + 10;
    static constexpr int off_misc = off_bar + n_bar * 8;  // tmem slot, abort flag, tile count
    static constexpr int total = off_misc + 16;
};

template <int D, bool BF16>
__global__ void __launch_bounds__(kFwdThreads, 1)
fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
           const __grid_constant__ CUtensorMap tmV, const FwdParams p) {
    using S = FwdSmem<D>;
    constexpr int NS = S::NS;
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    FA_TRACE_DECL

    const MaskArgs& mk = p.mask;
    const int nQ = mk.L.nQ;
    const int qb = nQ - 1 - int(blockIdx.x);  // long causal rows first
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / p.G;
    const int he = (mk.He == 1) ? 0 : h;

    uint16_t* list = reinterpret_cast<uint16_t*>(smem + S::off_list);
    volatile int* misc = reinterpret_cast<volatile int*>(smem + S::off_misc);  // [0] tmem, [1] abort, [2] T
    const uint32_t bar0 = sbase + S::off_bar;
    auto BAR = [&](int i) { return bar0 + 8u * uint32_t(i); };
    const int B_QFULL = 0, B_KFULL = 1, B_VFULL = 1 + NS, B_KEMPTY = 1 + 2 * NS, B_VEMPTY = 1 + 3 * NS,
              B_SFULL = 1 + 4 * NS, B_PHALF0 = B_SFULL + 2, B_PHALF1 = B_SFULL + 4, B_PVDONE = B_SFULL + 6, B_TURN = B_SFULL + 8;
    Abort ab{misc + 1, p.status};

    int lo, hi;
    kv_range(mk, b, he, qb, lo, hi);
    int n = hi - lo;
    if (n > kListCap) n = kListCap;  // the host refuses problems that could exceed the cap

    if (tid == 0) {
        mbar_init(BAR(B_QFULL), 1);
        for (int s = 0; s < NS; ++s) {
            mbar_init(BAR(B_KFULL + s), 1);
            mbar_init(BAR(B_VFULL + s), 1);
            mbar_init(BAR(B_KEMPTY + s), 1);
            mbar_init(BAR(B_VEMPTY + s), 1);
        }
        for (int w = 0; w < 2; ++w) {
            mbar_init(BAR(B_SFULL + w), 1);
            mbar_init(BAR(B_PHALF0 + w), 128);
            mbar_init(BAR(B_PHALF1 + w), 128);
            mbar_init(BAR(B_PVDONE + w), 1);
            mbar_init(BAR(B_TURN + w), 128);
        }
        misc[1] = (*reinterpret_cast<volatile int*>(p.status) != 0 || (sbase & 1023u) != 0) ? 1 : 0;
        misc[2] = 0;
        fence_mbar_init();
    }
    if (warp == 9) {
        tmem_alloc(sbase + S::off_misc, 512);
        tmem_relinquish();
    }
    // tile flags for [lo, lo+n)
    for (int i = tid; i < n; i += kFwdThreads) list[i] = uint16_t(classify_from_plan(mk, b, he, qb, lo + i));
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // compaction to the visited list: entry = (index relative to lo) | flags << 10
    if (warp == 0) {
        const int T = compact_visit_list(list, n, lane);
        if (lane == 0) misc[2] = T;
    }
    __syncthreads();
    const uint32_t tmem = uint32_t(misc[0]);
    const int T = misc[2];
    const bool aborted = misc[1] != 0;

    const uint32_t sQ = sbase + S::off_q;
    auto sK = [&](int s) { return sbase + S::off_k + uint32_t(s) * S::TILE; };
    auto sV = [&](int s) { return sbase + S::off_v + uint32_t(s) * S::TILE; };

    if (warp >= 8) {
        setmaxnreg_dec<72>();
        if (aborted || T == 0) {
            // nothing to load or multiply
        } else if (warp == 8) {
            // ------------------------------ TMA producer ------------------------------
            if (lane == 0) {
                tma_prefetch_desc(&tmQ);
                tma_prefetch_desc(&tmK);
                tma_prefetch_desc(&tmV);
                mbar_expect_tx(BAR(B_QFULL), S::TILE);
                for (int x = 0; x < S::NBOX; ++x)
                    tma_load_4d(sQ + x * S::BOX, &tmQ, BAR(B_QFULL), x * 64, qb * kBlk, h, b);
                bool ok = true;
                // K runs one tile ahead of V
                for (int t = 0; t <= T && ok; ++t) {
                    if (t < T) {
                        const int kb = lo + (list[t] & 1023);
                        const int st = t % NS, use = t / NS;
                        if (use > 0) ok = mbar_wait(BAR(B_KEMPTY + st), (use - 1) & 1, ab, ST_WAIT_TIMEOUT + 1);
                        if (!ok) break;
                        mbar_expect_tx(BAR(B_KFULL + st), S::TILE);
                        for (int x = 0; x < S::NBOX; ++x)
                            tma_load_4d(sK(st) + x * S::BOX, &tmK, BAR(B_KFULL + st), x * 64, kb * kBlk, hk, b);
                    }
                    if (t >= 1) {
                        const int tv = t - 1;
                        const int kb = lo + (list[tv] & 1023);
                        const int st = tv % NS, use = tv / NS;
                        if (use > 0) ok = mbar_wait(BAR(B_VEMPTY + st), (use - 1) & 1, ab, ST_WAIT_TIMEOUT + 2);
                        if (!ok) break;
                        mbar_expect_tx(BAR(B_VFULL + st), S::TILE);
                        for (int x = 0; x < S::NBOX; ++x)
                            tma_load_4d(sV(st) + x * S::BOX, &tmV, BAR(B_VFULL + st), x * 64, kb * kBlk, hk, b);
                    }
                }
            }
        } else if (warp == 9 || warp == 10) {
            // ------------------------------ MMA issuers ------------------------------
            // One issuing thread per softmax group: warp 9 owns the even visited tiles (S0 / O0),
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
                bool ok = mbar_wait(BAR(B_QFULL), 0, ab, ST_WAIT_TIMEOUT + 3);
                auto s_mmas = [&](int t) {
                    const int st = t % NS;
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {
                        const uint32_t off = uint32_t(kk >> 2) * S::BOX + uint32_t(kk & 3) * 32u;
                        umma_ss(tS, smem_desc_at(kDescKMajor, sQ + off), smem_desc_at(kDescKMajor, sK(st) + off),
                                idesc_s, kk > 0);
                    }
                    umma_commit(BAR(B_KEMPTY + st));
                    umma_commit(BAR(B_SFULL + w));
                    if (w == 0) FA_TRACE_EV(2, 2);
                };
                auto k_ready = [&](int t) {
                    return mbar_wait(BAR(B_KFULL + (t % NS)), (t / NS) & 1, ab, ST_WAIT_TIMEOUT + 4);
                };
                if (ok && w < T) {
                    ok = k_ready(w);
                    if (ok) { tc_fence_after(); s_mmas(w); }
                }
                int n_my = 0;
                for (int tp = w; tp < T && ok; tp += 2, ++n_my) {
                    const int st = tp % NS, use = tp / NS;
                    const bool more = tp + 2 < T;
                    ok = mbar_wait(BAR(B_VFULL + st), use & 1, ab, ST_WAIT_TIMEOUT + 5);
                    if (ok && more) ok = k_ready(tp + 2);
                    if (w == 0) FA_TRACE_EV(2, 3);
                    if (ok) ok = mbar_wait(BAR(B_PHALF0 + w), n_my & 1, ab, ST_WAIT_TIMEOUT + 6);
                    if (!ok) break;
                    tc_fence_after();
                    if (w == 0) FA_TRACE_EV(2, 4);
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        umma_ts(tO, tS + uint32_t(kk) * 8u, smem_desc_at(desc_v, sV(st) + uint32_t(kk) * 2048u), idesc_pv,
                                (n_my > 0 || kk > 0) ? 1u : 0u);
                    ok = mbar_wait(BAR(B_PHALF1 + w), n_my & 1, ab, ST_WAIT_TIMEOUT + 6);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int kk = 4; kk < 8; ++kk)
                        umma_ts(tO, tS + uint32_t(kk) * 8u, smem_desc_at(desc_v, sV(st) + uint32_t(kk) * 2048u), idesc_pv, 1u);
                    umma_commit(BAR(B_VEMPTY + st));
                    umma_commit(BAR(B_PVDONE + w));
                    if (w == 0) FA_TRACE_EV(2, 5);
                    if (more) s_mmas(tp + 2);
                }
            }
        }
        __syncwarp();
    } else {
        setmaxnreg_inc<216>();
        // ------------------------------ softmax groups ------------------------------
        const int w = warp >> 2;           // group
        const int r = tid & 127;           // row inside the block
        const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
        const int row = qb * kBlk + r;
        const float c = p.scale_log2;
        const int64_t bh_ids = int64_t(b) * mk.He + he;
        const int qc = (mk.mode == 1) ? mk.plan[mk.L.off_qc + bh_ids * mk.L.Mpad + row] : 0;
        float m_run = -INFINITY, l_run = 0.f;
        int n_my = 0;
        bool ok = !aborted;
        const uint32_t tS = tmem + lane_base + uint32_t(w) * 128u;
        const uint32_t tO = tmem + lane_base + 256u + uint32_t(w) * uint32_t(D);

        const int n_other = (w == 0) ? T / 2 : (T + 1) / 2;  // tiles of the other group
        if (w == 1 && T > 0 && ok) mbar_arrive(BAR(B_TURN + 0));  // group 0 takes the first turn
        for (int t = w; t < T && ok; t += 2, ++n_my) {
            const uint32_t entry = list[t];
            const uint32_t fl = entry >> 10;
            const int k0 = (lo + int(entry & 1023u)) * kBlk;
            if (r == 0) FA_TRACE_EV(w, 10);
            ok = mbar_wait(BAR(B_SFULL + w), n_my & 1, ab, ST_WAIT_TIMEOUT + 7);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            if (r == 0) FA_TRACE_EV(w, 11);
            uint32_t sr[128];
#pragma unroll
            for (int q = 0; q < 4; ++q) tmem_ld32(tS + uint32_t(q) * 32u, sr + q * 32);
            tc_wait_ld();
            float* s = reinterpret_cast<float*>(sr);
            if (r == 0) FA_TRACE_EV(w, 12);

            if (fl & (TILE_BOUND | TILE_DOC)) {
                int lim = kBlk - 1;
                if (fl & TILE_BOUND) {
                    int jmax = mk.N - 1;
                    if (mk.causal) jmax = min(jmax, row + mk.gap);
                    lim = jmax - k0;
                }
                if ((fl & TILE_DOC) && qc < 0) {
                    const int4* kc4 = reinterpret_cast<const int4*>(mk.plan + mk.L.off_kc + bh_ids * mk.L.Npad + k0);
#pragma unroll
                    for (int q = 0; q < 32; ++q) {
                        const int4 kc = __ldg(kc4 + q);
                        s[4 * q + 0] = (kc.x == qc && 4 * q + 0 <= lim) ? s[4 * q + 0] : -INFINITY;
                        s[4 * q + 1] = (kc.y == qc && 4 * q + 1 <= lim) ? s[4 * q + 1] : -INFINITY;
                        s[4 * q + 2] = (kc.z == qc && 4 * q + 2 <= lim) ? s[4 * q + 2] : -INFINITY;
                        s[4 * q + 3] = (kc.w == qc && 4 * q + 3 <= lim) ? s[4 * q + 3] : -INFINITY;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 128; ++j) s[j] = (j <= lim) ? s[j] : -INFINITY;
                }
            }
            if (r == 0) FA_TRACE_EV(w, 18);
            float mxa[8];
#pragma unroll
            for (int a = 0; a < 8; ++a) mxa[a] = max3(s[a], s[8 + a], s[16 + a]);
#pragma unroll
            for (int j = 24; j < 120; j += 16) {
#pragma unroll
                for (int a = 0; a < 8; ++a) mxa[a] = max3(mxa[a], s[j + a], s[j + 8 + a]);
            }
#pragma unroll
            for (int a = 0; a < 8; ++a) mxa[a] = fmaxf(mxa[a], s[120 + a]);
            const float mx = fmaxf(max3(mxa[0], mxa[1], mxa[2]), max3(max3(mxa[3], mxa[4], mxa[5]), mxa[6], mxa[7]));
            if (r == 0) FA_TRACE_EV(w, 19);
            float m_new = fmaxf(m_run, mx);
            // lazy rescale: keep the old reference point while the new maximum is within 2^8 of it
            const bool need = (m_new - m_run) * c > 8.0f;
            if (!need) m_new = m_run;
            if (__any_sync(0xffffffffu, need)) {
                const float alpha = need ? fast_exp2((m_run - m_new) * c) : 1.0f;
                l_run *= alpha;
                if (n_my > 0) {
                    ok = mbar_wait(BAR(B_PVDONE + w), (n_my - 1) & 1, ab, ST_WAIT_TIMEOUT + 8);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int q = 0; q < D / 32; ++q) {
                        uint32_t orr[32];
                        tmem_ld32(tO + uint32_t(q) * 32u, orr);
                        tc_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; ++j) orr[j] = __float_as_uint(__uint_as_float(orr[j]) * alpha);
                        tmem_st32(tO + uint32_t(q) * 32u, orr);
                    }
                    tc_wait_st();
                }
            }
            if (r == 0) FA_TRACE_EV(w, 13);
            m_run = m_new;
            const float mneg = (m_run == -INFINITY) ? 0.f : -m_run * c;
            // exp2(s*c - m*c) on packed pairs; P goes to TMEM in two halves so that the first four
            // k-steps of P*V can start while the second half is still being exponentiated. MUFU
            // (16 ex2 per clock and SM) is as scarce as the tensor pipe here, so on tiles without
            // masked entries kPolyOf4 of every 4 pairs are evaluated on the FMA pipe instead.
            const uint64_t c2 = pack_f2(c, c), mneg2 = pack_f2(mneg, mneg);
            uint64_t lacc0 = pack_f2(0.f, 0.f), lacc1 = lacc0;
            // The exp phase is taken in turns (barriers turn[0], turn[1]; group 0 first): left alone,
            // the groups fall into lockstep, exponentiate together at half MUFU rate each and then
            // queue their MMAs together, which halves the use of both pipes. In turns, one group
            // exponentiates while the other group's P*V and next S run on the tensor pipe.
            ok = mbar_wait(BAR(B_TURN + w), n_my & 1, ab, ST_WAIT_TIMEOUT + 10);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const bool poly_ok = (fl & (TILE_BOUND | TILE_DOC)) == 0;
            auto exp_half = [&](auto use_poly, int half) {
#pragma unroll
                for (int q = 2 * half; q < 2 * half + 2; ++q) {
                    uint32_t pk[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const uint64_t x2 = fma_f2(pack_f2(s[32 * q + 2 * j], s[32 * q + 2 * j + 1]), c2, mneg2);
                        float p0, p1;
                        if (decltype(use_poly)::value && (j & 3) < kPolyOf4) {
                            exp2_poly2(x2, p0, p1);
                        } else {
                            float x0, x1;
                            unpack_f2(x2, x0, x1);
                            p0 = fast_exp2(x0);
                            p1 = fast_exp2(x1);
                        }
                        if (j & 1) lacc1 = add_f2(lacc1, pack_f2(p0, p1)); else lacc0 = add_f2(lacc0, pack_f2(p0, p1));
                        pk[j] = pack2<BF16>(p0, p1);
                    }
                    tmem_st16(tS + uint32_t(q) * 16u, pk);
                }
                tc_wait_st();
                tc_fence_before();
                mbar_arrive(BAR((half ? B_PHALF1 : B_PHALF0) + w));
                if (r == 0) FA_TRACE_EV(w, 14 + half);
            };
            if (poly_ok) {
                exp_half(std::true_type{}, 0);
                exp_half(std::true_type{}, 1);
            } else {
                exp_half(std::false_type{}, 0);
                exp_half(std::false_type{}, 1);
            }
            // hand the turn over, unless the other group has no tile left to take it for
            if (w == 0 ? (n_my < n_other) : (n_my + 1 < n_other)) mbar_arrive(BAR(B_TURN + (w ^ 1)));
            {
                float a0, a1, b0, b1;
                unpack_f2(lacc0, a0, a1);
                unpack_f2(lacc1, b0, b1);
                l_run += (a0 + a1) + (b0 + b1);
            }
            if (r == 0) FA_TRACE_EV(w, 15);
        }

        // ------------------------------ epilogue ------------------------------
        // wait for this group's last P*V, then merge the two partial softmaxes
        if (ok && n_my > 0) {
            ok = mbar_wait(BAR(B_PVDONE + w), (n_my - 1) & 1, ab, ST_WAIT_TIMEOUT + 9);
        }
        ok = __all_sync(0xffffffffu, ok);
        // Group 0 owns tile 0, so once both groups have passed this barrier every MMA of the CTA
        // has completed and the Q tile may be reused as the exchange buffer. (A group without
        // tiles gets here at once; it must not touch Q before the barrier.)
        tc_fence_before();
        named_bar_sync(1, 256);
        tc_fence_after();
        float* ml = reinterpret_cast<float*>(smem + S::off_q);  // [2 groups][m, l][128]
        if (T > 0 && !aborted) {
            ml[(w * 2 + 0) * 128 + r] = m_run;
            ml[(w * 2 + 1) * 128 + r] = l_run;
        }
        named_bar_sync(1, 256);
        const bool healthy = ok && (misc[1] == 0);
        if (healthy) {
            float m0 = -INFINITY, l0 = 0.f, m1 = -INFINITY, l1 = 0.f;
            if (T > 0) {
                m0 = ml[0 * 128 + r]; l0 = ml[1 * 128 + r];
                m1 = ml[2 * 128 + r]; l1 = ml[3 * 128 + r];
            }
            const float mt = fmaxf(m0, m1);
            const float a0 = (m0 == -INFINITY) ? 0.f : fast_exp2((m0 - mt) * c);
            const float a1 = (m1 == -INFINITY) ? 0.f : fast_exp2((m1 - mt) * c);
            const float lt = l0 * a0 + l1 * a1;
            const float inv = (lt > 0.f) ? 1.0f / lt : 0.f;
            const float f0 = a0 * inv, f1 = a1 * inv;
            const bool use0 = (T > 0) && (f0 != 0.f), use1 = (T > 1) && (f1 != 0.f);
            if (w == 0) {
                const float lse = (lt > 0.f) ? fmaf(mt, c, log2f(lt)) : -INFINITY;
                p.lse[(int64_t(b) * p.H + h) * mk.L.Mpad + row] = lse;
            }
            constexpr int HALF = D / 2;
            const uint32_t c0 = uint32_t(w) * HALF;
            uint8_t* orow = static_cast<uint8_t*>(p.o.ptr) +
                            2 * (int64_t(b) * p.o.sb + int64_t(h) * p.o.sh + int64_t(row) * p.o.sl + c0);
#pragma unroll
            for (int q = 0; q < HALF / 32; ++q) {
                uint32_t x0[32], x1[32];
                // tcgen05.ld is warp-collective: always executed, the values are ignored when unused
                tmem_ld32(tmem + lane_base + 256u + c0 + uint32_t(q) * 32u, x0);
                tmem_ld32(tmem + lane_base + 256u + uint32_t(D) + c0 + uint32_t(q) * 32u, x1);
                tc_wait_ld();
                uint32_t out[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    float v0 = 0.f, v1 = 0.f;
                    if (use0) {
                        v0 = __uint_as_float(x0[2 * j]) * f0;
                        v1 = __uint_as_float(x0[2 * j + 1]) * f0;
                    }
                    if (use1) {
                        v0 = fmaf(__uint_as_float(x1[2 * j]), f1, v0);
                        v1 = fmaf(__uint_as_float(x1[2 * j + 1]), f1, v1);
                    }
                    out[j] = pack2<BF16>(v0, v1);
                }
                if (row < mk.M) {
                    uint4* dst = reinterpret_cast<uint4*>(orow + q * 64);
#pragma unroll
                    for (int j = 0; j < 4; ++j) dst[j] = make_uint4(out[4 * j], out[4 * j + 1], out[4 * j + 2], out[4 * j + 3]);
                }
            }
        }
    }

    // ------------------------------ tear-down ------------------------------
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

// ---- host launcher (called from api.cu) -------------------------------------------------
template <int D, bool BF16>
static cudaError_t launch_fwd_t(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                                const FwdParams& p, int B, cudaStream_t stream) {
    auto kern = fwd_kernel<D, BF16>;
    constexpr int smem = FwdSmem<D>::total;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    dim3 grid(p.mask.L.nQ, p.H, B);
    kern<<<grid, kFwdThreads, smem, stream>>>(tq, tk, tv, p);
    return cudaGetLastError();
}

FA_TRACE_DUMP_FN(fa_trace_dump_fwd)

cudaError_t launch_fwd(int D, bool bf16, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                       const FwdParams& p, int B, cudaStream_t stream) {
    if (D == 128) return bf16 ? launch_fwd_t<128, true>(tq, tk, tv, p, B, stream)
                              : launch_fwd_t<128, false>(tq, tk, tv, p, B, stream);
    return bf16 ? launch_fwd_t<64, true>(tq, tk, tv, p, B, stream) : launch_fwd_t<64, false>(tq, tk, tv, p, B, stream);
}

}  // namespace fa
