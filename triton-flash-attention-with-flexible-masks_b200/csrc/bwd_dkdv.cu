// dK / dV kernel. Replaces `_bwd_kv_kernel` (flash_triton.py:175-321) and the grouped-query
// sum that follows it (:635-637): per block of 128 keys, walk the visited query tiles of every
// query head of the group, recompute P, and accumulate dV += P^T dO, dK += dS^T Q in fp32.
//
// The tile is kept transposed (rows = keys, columns = queries): S^T = K Q^T and dP^T = V dO^T
// land in TMEM with one key per lane, so P^T and dS^T (input dtype) can be written back to
// TMEM and used directly as the A operand of the dV / dK MMAs, with dO / Q read from shared
// memory as MN-major B operands. One CTA = one key block of one (batch, kv head), 12 warps:
//   warps 0-7  two compute groups; thread r of group g owns key row r and query columns
//              [64g, 64g+64) of every tile
//   warp 8     TMA producer (K, V once; Q ring with the per-row LSE / delta / id codes; dO ring)
//   warps 9,10 tcgen05.mma issuers (warp 9 also owns the TMEM allocation)
// TMEM columns: S^T [0,128)  dP^T [128,256)  dV [256,256+D)  dK [256+D,256+2D).
#include "common.cuh"
#include "params.cuh"
#include "trace.cuh"

namespace fa {

template <int D>
struct DkdvSmem {
    static constexpr int NST = (D == 128) ? 2 : 4;
    static constexpr int TILE = kBlk * D * 2;
    static constexpr int BOX = kBlk * 64 * 2;
    static constexpr int NBOX = D / 64;
    static constexpr int VEC = 3 * kBlk * 4;  // lse, delta, query codes of one query block
    static constexpr int off_k = 0;
    static constexpr int off_v = TILE;
    static constexpr int off_q = 2 * TILE;
    static constexpr int off_do = off_q + NST * TILE;
    static constexpr int off_vec = off_do + NST * TILE;
    static constexpr int off_list = off_vec + NST * VEC;
    static constexpr int off_bar = off_list + kListCap * 2;
    // kv_full, q_full[NST], do_full[NST], q_empty[NST], do_empty[NST], s_full, dp_full, p_full, ds_full, done
    static constexpr int n_bar = 1 + 4 * NST + 5;
    static constexpr int off_misc = off_bar + n_bar * 8;
    static constexpr int total = off_misc + 16;
};

// Flags of tile (qb, kb) for all query heads of one kv head at once. When the heads disagree
// (ids given per head) the id check is forced, which is always exact.
__device__ __forceinline__ uint32_t classify_group(const MaskArgs& mk, int b, int hk, int G, int qb, int kb) {
    if (mk.He == 1 || G == 1) return classify_from_plan(mk, b, mk.He == 1 ? 0 : hk * G, qb, kb);
    uint32_t f = 0;
    bool all = true;
    for (int g = 0; g < G; ++g) {
        const uint32_t fg = classify_from_plan(mk, b, hk * G + g, qb, kb);
        if (fg & TILE_VISIT) f |= fg; else all = false;
    }
    if (f && !all) f |= TILE_DOC;
    return f;
}

template <int D, bool BF16>
__global__ void __launch_bounds__(kAttnThreads, 1)
bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                const DkdvParams p) {
    using S = DkdvSmem<D>;
    constexpr int NST = S::NST;
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    FA_TRACE_DECL

    const MaskArgs& mk = p.mask;
    const int kb = blockIdx.x;  // with a causal mask the first key blocks are the long ones
    const int hk = blockIdx.y, b = blockIdx.z;
    const int G = p.G;

    uint16_t* list = reinterpret_cast<uint16_t*>(smem + S::off_list);
    volatile int* misc = reinterpret_cast<volatile int*>(smem + S::off_misc);
    const uint32_t bar0 = sbase + S::off_bar;
    auto BAR = [&](int i) { return bar0 + 8u * uint32_t(i); };
    const int B_KV = 0, B_QFULL = 1, B_DOFULL = B_QFULL + NST, B_QEMPTY = B_DOFULL + NST, B_DOEMPTY = B_QEMPTY + NST,
              B_SFULL = B_DOEMPTY + NST, B_DPFULL = B_SFULL + 1, B_PFULL = B_SFULL + 2, B_DSFULL = B_SFULL + 3,
              B_DONE = B_SFULL + 4;
    Abort ab{misc + 1, p.status};

    // union of the query-block ranges of the group's heads
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

    if (tid == 0) {
        mbar_init(BAR(B_KV), 1);
        for (int s = 0; s < NST; ++s) {
            mbar_init(BAR(B_QFULL + s), 1); mbar_init(BAR(B_DOFULL + s), 1);
            mbar_init(BAR(B_QEMPTY + s), 2); mbar_init(BAR(B_DOEMPTY + s), 2);  // one commit per MMA issuer
        }
        mbar_init(BAR(B_SFULL), 1);
        mbar_init(BAR(B_DPFULL), 1);
        mbar_init(BAR(B_PFULL), 256);
        mbar_init(BAR(B_DSFULL), 256);
        mbar_init(BAR(B_DONE), 2);
        misc[1] = (*reinterpret_cast<volatile int*>(p.status) != 0 || (sbase & 1023u) != 0) ? 1 : 0;
        misc[2] = 0;
        fence_mbar_init();
    }
    if (warp == 9) {
        tmem_alloc(sbase + S::off_misc, 512);
        tmem_relinquish();
    }
    for (int i = tid; i < n; i += kAttnThreads) list[i] = uint16_t(classify_group(mk, b, hk, G, lo + i, kb));
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) {
        const int Tn = compact_visit_list(list, n, lane);
        if (lane == 0) misc[2] = Tn;
    }
    __syncthreads();
    const uint32_t tmem = uint32_t(misc[0]);
    const int T = misc[2];
    const int NIT = T * G;  // tiles of all query heads of the group, head-major
    const bool aborted = misc[1] != 0;

    const uint32_t sK = sbase + S::off_k, sV = sbase + S::off_v;
    auto sQ = [&](int s) { return sbase + S::off_q + uint32_t(s) * S::TILE; };
    auto sdO = [&](int s) { return sbase + S::off_do + uint32_t(s) * S::TILE; };
    auto sVec = [&](int s) { return sbase + S::off_vec + uint32_t(s) * S::VEC; };

    if (warp >= 8) {
        setmaxnreg_dec<56>();
        if (aborted || NIT == 0) {
        } else if (warp == 8) {
            // ------------------------------ TMA producer ------------------------------
            if (lane == 0) {
                tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmdO); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
                mbar_expect_tx(BAR(B_KV), 2 * S::TILE);
                for (int x = 0; x < S::NBOX; ++x) {
                    tma_load_4d(sK + x * S::BOX, &tmK, BAR(B_KV), x * 64, kb * kBlk, hk, b);
                    tma_load_4d(sV + x * S::BOX, &tmV, BAR(B_KV), x * 64, kb * kBlk, hk, b);
                }
                bool ok = true;
                const uint32_t vec_bytes = (mk.mode == 1) ? 3u * kBlk * 4u : 2u * kBlk * 4u;
                for (int it = 0; it < NIT && ok; ++it) {
                    const int g = it / T, idx = it - g * T;
                    const int h = hk * G + g;
                    const int qb = lo + (list[idx] & 1023);
                    const int st = it % NST, use = it / NST;
                    if (use > 0) ok = mbar_wait(BAR(B_QEMPTY + st), (use - 1) & 1, ab, ST_WAIT_TIMEOUT + 41);
                    if (!ok) break;
                    mbar_expect_tx(BAR(B_QFULL + st), S::TILE + vec_bytes);
                    for (int x = 0; x < S::NBOX; ++x)
                        tma_load_4d(sQ(st) + x * S::BOX, &tmQ, BAR(B_QFULL + st), x * 64, qb * kBlk, h, b);
                    const int64_t roff = (int64_t(b) * p.H + h) * mk.L.Mpad + int64_t(qb) * kBlk;
                    bulk_load_1d(sVec(st), p.lse + roff, kBlk * 4, BAR(B_QFULL + st));
                    bulk_load_1d(sVec(st) + kBlk * 4, p.delta + roff, kBlk * 4, BAR(B_QFULL + st));
                    if (mk.mode == 1) {
                        const int he = (mk.He == 1) ? 0 : h;
                        const int32_t* qc = mk.plan + mk.L.off_qc + (int64_t(b) * mk.He + he) * mk.L.Mpad + int64_t(qb) * kBlk;
                        bulk_load_1d(sVec(st) + 2 * kBlk * 4, qc, kBlk * 4, BAR(B_QFULL + st));
                    }
                    if (use > 0) ok = mbar_wait(BAR(B_DOEMPTY + st), (use - 1) & 1, ab, ST_WAIT_TIMEOUT + 42);
                    if (!ok) break;
                    mbar_expect_tx(BAR(B_DOFULL + st), S::TILE);
                    for (int x = 0; x < S::NBOX; ++x)
                        tma_load_4d(sdO(st) + x * S::BOX, &tmdO, BAR(B_DOFULL + st), x * 64, qb * kBlk, h, b);
                }
            }
        } else if (warp == 9 || warp == 10) {
            // ------------------------------ MMA issuers ------------------------------
            // Two issuing threads, so that neither the blocking tcgen05.mma issue nor the barrier
            // round trips of one pair of GEMMs delay the other pair:
            //   warp 9 : dV(it) += P^T dO, then S^T(it+1) = K Q^T  (S^T overwrites P^T: same thread, in order)
            //   warp 10: dK(it) += dS^T Q, then dP^T(it+1) = V dO^T (dP^T overwrites dS^T: same thread)
            // Each Q / dO stage is read by both threads, so its "empty" barrier takes two commits.
            if (lane == 0) {
                const bool is_a = (warp == 9);
                constexpr uint32_t idesc_s = make_idesc(BF16, 128, 128, false, false);
                constexpr uint32_t idesc_d = make_idesc(BF16, 128, D, false, true);
                constexpr uint64_t desc_mn = desc_mn_major(S::BOX);
                bool ok = mbar_wait(BAR(B_KV), 0, ab, ST_WAIT_TIMEOUT + 43);
                auto q_ready = [&](int it) { return mbar_wait(BAR(B_QFULL + it % NST), (it / NST) & 1, ab, ST_WAIT_TIMEOUT + 44); };
                auto do_ready = [&](int it) { return mbar_wait(BAR(B_DOFULL + it % NST), (it / NST) & 1, ab, ST_WAIT_TIMEOUT + 45); };
                auto ss_mmas = [&](uint32_t d, uint32_t a_tile, uint32_t b_tile) {
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {
                        const uint32_t off = uint32_t(kk >> 2) * S::BOX + uint32_t(kk & 3) * 32u;
                        umma_ss(d, smem_desc_at(kDescKMajor, a_tile + off), smem_desc_at(kDescKMajor, b_tile + off),
                                idesc_s, kk > 0);
                    }
                };
                auto acc_mmas = [&](int it, uint32_t a_base, uint32_t d, uint32_t b_tile) {
#pragma unroll
                    for (int kk = 0; kk < kBlk / 16; ++kk) {
                        const uint32_t acol = (kk < 4) ? uint32_t(kk) * 8u : 64u + uint32_t(kk - 4) * 8u;
                        umma_ts(d, a_base + acol, smem_desc_at(desc_mn, b_tile + uint32_t(kk) * 2048u), idesc_d,
                                (it > 0 || kk > 0) ? 1u : 0u);
                    }
                };
                if (is_a) {
                    if (ok) ok = q_ready(0);
                    if (ok) {
                        tc_fence_after();
                        ss_mmas(tmem, sK, sQ(0));  // S^T(0)
                        umma_commit(BAR(B_QEMPTY + 0));
                        umma_commit(BAR(B_SFULL));
                    }
                    for (int it = 0; it < NIT && ok; ++it) {
                        const int st = it % NST;
                        const bool more = it + 1 < NIT;
                        ok = do_ready(it);
                        FA_TRACE_EV(2, 3);
                        if (ok) ok = mbar_wait(BAR(B_PFULL), it & 1, ab, ST_WAIT_TIMEOUT + 46);
                        if (!ok) break;
                        tc_fence_after();
                        FA_TRACE_EV(2, 4);
                        acc_mmas(it, tmem, tmem + 256u, sdO(st));  // dV += P^T dO
                        umma_commit(BAR(B_DOEMPTY + st));
                        // Q(it+1) can only be loaded once dK(it-1) has released its stage, so it is
                        // waited for here and not ahead of P(it)
                        if (more) ok = q_ready(it + 1);
                        if (ok && more) {
                            tc_fence_after();
                            ss_mmas(tmem, sK, sQ((it + 1) % NST));
                            umma_commit(BAR(B_QEMPTY + (it + 1) % NST));
                            umma_commit(BAR(B_SFULL));
                        }
                        FA_TRACE_EV(2, 2);
                    }
                } else {
                    if (ok) ok = do_ready(0);
                    if (ok) {
                        tc_fence_after();
                        ss_mmas(tmem + 128u, sV, sdO(0));  // dP^T(0)
                        umma_commit(BAR(B_DOEMPTY + 0));
                        umma_commit(BAR(B_DPFULL));
                    }
                    for (int it = 0; it < NIT && ok; ++it) {
                        const int st = it % NST;
                        const bool more = it + 1 < NIT;
                        ok = q_ready(it);
                        if (ok && more) ok = do_ready(it + 1);
                        if (ok) ok = mbar_wait(BAR(B_DSFULL), it & 1, ab, ST_WAIT_TIMEOUT + 47);
                        // S^T(it+1) gates the next P and must not share the tensor pipe with this
                        // batch (the pipe serves both issuers in turn): let it finish first
                        if (ok && more) ok = mbar_wait(BAR(B_SFULL), (it + 1) & 1, ab, ST_WAIT_TIMEOUT + 49);
                        if (!ok) break;
                        tc_fence_after();
                        acc_mmas(it, tmem + 128u, tmem + 256u + uint32_t(D), sQ(st));  // dK += dS^T Q
                        umma_commit(BAR(B_QEMPTY + st));
                        if (more) {
                            ss_mmas(tmem + 128u, sV, sdO((it + 1) % NST));
                            umma_commit(BAR(B_DOEMPTY + (it + 1) % NST));
                            umma_commit(BAR(B_DPFULL));
                        }
                    }
                }
                if (ok) umma_commit(BAR(B_DONE));
            }
        }
        __syncwarp();
    } else {
        setmaxnreg_inc<224>();
        // ------------------------------ compute groups ------------------------------
        const int w = warp >> 2;
        const int r = tid & 127;
        const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
        const int j = kb * kBlk + r;  // this thread's key
        const int cbase = 64 * w;     // first query column of this thread inside a tile
        const float c = p.scale_log2;
        bool ok = !aborted;
        const uint32_t tS = tmem + lane_base + uint32_t(cbase);
        const uint32_t tdP = tmem + lane_base + 128u + uint32_t(cbase);

        for (int it = 0; it < NIT && ok; ++it) {
            const int g = it / T, idx = it - g * T;
            const int he = (mk.He == 1) ? 0 : hk * G + g;
            const uint32_t entry = list[idx];
            const uint32_t fl = entry >> 10;
            const int q0 = (lo + int(entry & 1023u)) * kBlk + cbase;  // first query row of this thread's columns
            const int st = it % NST;
            const float* vlse = reinterpret_cast<const float*>(smem + S::off_vec + st * S::VEC) + cbase;
            const float* vdelta = vlse + kBlk;
            const int* vqc = reinterpret_cast<const int*>(vlse + 2 * kBlk);

            if (r == 0) FA_TRACE_EV(w, 10);
            ok = mbar_wait(BAR(B_QFULL + st), (it / NST) & 1, ab, ST_WAIT_TIMEOUT + 48);
            if (ok) ok = mbar_wait(BAR(B_SFULL), it & 1, ab, ST_WAIT_TIMEOUT + 49);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            if (r == 0) FA_TRACE_EV(w, 11);
            uint32_t sr[64];
            tmem_ld32(tS, sr);
            tmem_ld32(tS + 32u, sr + 32);
            tc_wait_ld();
            if (r == 0) FA_TRACE_EV(w, 12);
            float* pr = reinterpret_cast<float*>(sr);
            {
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
            if (fl & (TILE_BOUND | TILE_DOC | TILE_QTAIL)) {
                int cmin = -0x40000000, cmax = 64;  // keep iff cmin <= column < cmax
                if ((fl & TILE_BOUND) && mk.causal) cmin = (j - mk.gap) - q0;
                if (fl & TILE_QTAIL) cmax = mk.M - q0;
                if (fl & TILE_DOC) {
                    const int kc = mk.plan[mk.L.off_kc + (int64_t(b) * mk.He + he) * mk.L.Npad + j];
#pragma unroll
                    for (int q = 0; q < 16; ++q) {
                        const int4 qc = *reinterpret_cast<const int4*>(vqc + 4 * q);
                        pr[4 * q + 0] = ((qc.x >= 0 || qc.x == kc) && 4 * q + 0 >= cmin && 4 * q + 0 < cmax) ? pr[4 * q + 0] : 0.f;
                        pr[4 * q + 1] = ((qc.y >= 0 || qc.y == kc) && 4 * q + 1 >= cmin && 4 * q + 1 < cmax) ? pr[4 * q + 1] : 0.f;
                        pr[4 * q + 2] = ((qc.z >= 0 || qc.z == kc) && 4 * q + 2 >= cmin && 4 * q + 2 < cmax) ? pr[4 * q + 2] : 0.f;
                        pr[4 * q + 3] = ((qc.w >= 0 || qc.w == kc) && 4 * q + 3 >= cmin && 4 * q + 3 < cmax) ? pr[4 * q + 3] : 0.f;
                    }
                } else {
#pragma unroll
                    for (int x = 0; x < 64; ++x) pr[x] = (x >= cmin && x < cmax) ? pr[x] : 0.f;
                }
            }
            uint32_t pk[32];
#pragma unroll
            for (int x = 0; x < 32; ++x) pk[x] = pack2<BF16>(pr[2 * x], pr[2 * x + 1]);
            tmem_st32(tS, pk);
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(BAR(B_PFULL));
            if (r == 0) FA_TRACE_EV(w, 15);

            ok = mbar_wait(BAR(B_DPFULL), it & 1, ab, ST_WAIT_TIMEOUT + 50);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            if (r == 0) FA_TRACE_EV(w, 16);
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
            if (r == 0) FA_TRACE_EV(w, 17);
        }

        // ------------------------------ epilogue ------------------------------
        if (ok && NIT > 0) ok = mbar_wait(BAR(B_DONE), 0, ab, ST_WAIT_TIMEOUT + 51);
        ok = __all_sync(0xffffffffu, ok);
        tc_fence_after();
        if (ok && misc[1] == 0) {
            constexpr int HALF = D / 2;
            const uint32_t c0 = uint32_t(w) * HALF;
#pragma unroll
            for (int which = 0; which < 2; ++which) {  // 0: dV, 1: dK
                const OutTensor& out = which ? p.dk : p.dv;
                const float mul = which ? p.sm_scale : 1.0f;  // flash_triton.py:313
                uint8_t* orow = static_cast<uint8_t*>(out.ptr) +
                                2 * (int64_t(b) * out.sb + int64_t(hk) * out.sh + int64_t(j) * out.sl + c0);
#pragma unroll
                for (int q = 0; q < HALF / 32; ++q) {
                    uint32_t x[32];
                    tmem_ld32(tmem + lane_base + 256u + uint32_t(which * D) + c0 + uint32_t(q) * 32u, x);
                    tc_wait_ld();
                    uint32_t o16[16];
#pragma unroll
                    for (int y = 0; y < 16; ++y) {
                        const float v0 = (NIT > 0) ? __uint_as_float(x[2 * y]) * mul : 0.f;
                        const float v1 = (NIT > 0) ? __uint_as_float(x[2 * y + 1]) * mul : 0.f;
                        o16[y] = pack2<BF16>(v0, v1);
                    }
                    if (j < mk.N) {
                        uint4* dst = reinterpret_cast<uint4*>(orow + q * 64);
#pragma unroll
                        for (int y = 0; y < 4; ++y) dst[y] = make_uint4(o16[4 * y], o16[4 * y + 1], o16[4 * y + 2], o16[4 * y + 3]);
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

template <int D, bool BF16>
static cudaError_t launch_dkdv_t(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                                 const CUtensorMap& tdo, const DkdvParams& p, int B, cudaStream_t stream) {
    auto kern = bwd_dkdv_kernel<D, BF16>;
    constexpr int smem = DkdvSmem<D>::total;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    dim3 grid(p.mask.L.nK, p.Hk, B);
    kern<<<grid, kAttnThreads, smem, stream>>>(tq, tk, tv, tdo, p);
    return cudaGetLastError();
}

FA_TRACE_DUMP_FN(fa_trace_dump_dkdv)

cudaError_t launch_bwd_dkdv(int D, bool bf16, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                            const CUtensorMap& tdo, const DkdvParams& p, int B, cudaStream_t stream) {
    if (D == 128) return bf16 ? launch_dkdv_t<128, true>(tq, tk, tv, tdo, p, B, stream)
                              : launch_dkdv_t<128, false>(tq, tk, tv, tdo, p, B, stream);
    return bf16 ? launch_dkdv_t<64, true>(tq, tk, tv, tdo, p, B, stream)
                : launch_dkdv_t<64, false>(tq, tk, tv, tdo, p, B, stream);
}

}  // namespace fa
