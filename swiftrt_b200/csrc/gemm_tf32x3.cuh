// Float32 products whose streamed operand is read from HBM exactly once: a CTA-pair kernel
// (tcgen05 cta_group::2, 256 x 256 tiles) that multiplies
//     a . b  ~  hi(a) . hi(b)                      one TF32 pass over the raw fp32 tiles
//             + lo(a) . b16(b) + b16(a) . lo(b)    one BFloat16 pass over "correction" tiles
// where hi(x) is x with its low 13 mantissa bits cleared (what a TF32 MMA reads from an fp32 word),
// lo(x) = x - hi(x) (exact, at most 13 significant bits) and b16 is the BFloat16 rounding.  The
// correction terms are 2^-11 of the product, so 8 significant bits of each factor keep them to
// 2^-19 of the product, and a BFloat16 MMA costs half a TF32 one: the whole product costs two TF32
// passes instead of the three of gemm_tcgen05_split_kernel.  The dropped lo . lo term is 2^-22.
//
// Operands.  op(a) [M x K] must be K-contiguous; it is streamed by TMA as raw fp32 (the TF32 operand)
// and the worker warps of each CTA write the BFloat16 tile  [ lo(a) | b16(a) ]  (32 + 32 values = one
// 128-byte swizzled row per A row and k-block) beside it.  op(b) is the small, re-used operand: a
// pre-pass (tf32x3_pack_kernel) writes it once per call as  Bh = fp32 [N x Kp]  (K-contiguous, zero
// padded to whole k-blocks) and  Bc = bf16 [N x 2 Kp]  holding  [ b16(b) | lo(b) ]  per k-block, so
// that both of its tiles arrive by TMA and one K = 64 BFloat16 MMA chain computes both correction
// terms at once.  Both accumulators (main, corrections) live in TMEM (2 x 256 columns) and are added
// by the epilogue; keeping the small terms apart matters because the accumulator add truncates.
//
//   warp 0      TMA producer (both CTAs): A tile -> own fullA[s]; Bh and Bc half tiles -> the leader's fullB[s]
//   warp 1      MMA issuer (leader CTA only) and TMEM owner
//   warps 2-9   workers: during the reduction fullA[s] -> write [lo | b16] -> arrive on the leader's ready[s]
//               (count 16); after the tile's last MMA the same warps are the epilogue
//   empty[s]    both CTAs, one multicast commit of the leader frees the stage in both
//
// Non-finite inputs: lo(x) = x for an infinity or NaN, and a zero low part of a non-zero value is
// replaced by x 2^-30 (far below the dropped term), so that infinity times a value whose low part
// vanishes gives the infinity of the reference loop instead of inf . 0 = NaN.
#pragma once
#include "gemm_tcgen05.cuh"

namespace srt {

// Two shapes of the same kernel.
//   BN = 256: 64 KB stages (three fit), both accumulators fill TMEM: eight "worker" warps write the correction
//             tiles during the reduction and drain the accumulators afterwards (the epilogue is exposed).
//             The default: measured faster (141 us against 161 us on 65536 x 1024 . 1024 x 256).
//   BN = 128: 48 KB stages (four fit), accumulators double-buffered: eight transform warps and four epilogue
//             warps, the epilogue of one tile runs under the reduction of the next; twice the MMA
//             instructions and operand reads per flop.
constexpr uint32_t kX3TransformWarps = 8;
constexpr uint32_t kX3TileBytes = 128 * kRowBytes;                     // one 128-row, 128-byte-wide tile: 16 KB
__host__ __device__ constexpr uint32_t x3_stage_bytes(uint32_t bn) { return 2 * kX3TileBytes + bn * kRowBytes; }   // A raw, A corrections, Bh half, Bc half
__host__ __device__ constexpr uint32_t x3_stages(uint32_t bn) { return bn == 128 ? 4u : 3u; }
__host__ __device__ constexpr uint32_t x3_epilogue_warps(uint32_t bn) { return bn == 128 ? 4u : 8u; }
__host__ __device__ constexpr uint32_t x3_threads(uint32_t bn) { return bn == 128 ? (2 + 4 + kX3TransformWarps) * 32 : (2 + 8) * 32; }
__host__ __device__ constexpr uint32_t x3_smem_bytes(uint32_t bn) { return x3_stages(bn) * x3_stage_bytes(bn) + x3_epilogue_warps(bn) * 4096 + 1024; }
constexpr uint32_t kX3MaxStages = 4;

struct PackParams {
    const float* b;                 // op(b) element (n, k) at b + batch b_b + n b_n + k b_k
    long long b_b, b_n, b_k;
    float* bh;                      // [batch][N][Kp]
    __nv_bfloat16* bc;              // [batch][N][2 Kp]
    uint32_t N, K, Kp, batch;
};

// One thread per (n, 4 consecutive k): reads along whichever of n, k is contiguous in memory.
__global__ void __launch_bounds__(256)
tf32x3_pack_kernel(const PackParams p)
{
    launch_dependents();          // the product kernel may start its prologue; it waits before reading Bh / Bc
    const uint32_t kq = p.Kp / 4;
    const unsigned long long total = static_cast<unsigned long long>(p.batch) * p.N * kq;
    const bool k_fast = p.b_k == 1 || p.b_n != 1;
    for (unsigned long long i = blockIdx.x * 256ull + threadIdx.x; i < total; i += gridDim.x * 256ull) {
        uint32_t n, q, bt;
        if (k_fast) { q = static_cast<uint32_t>(i % kq); n = static_cast<uint32_t>((i / kq) % p.N); bt = static_cast<uint32_t>(i / (static_cast<unsigned long long>(kq) * p.N)); }
        else        { n = static_cast<uint32_t>(i % p.N); q = static_cast<uint32_t>((i / p.N) % kq); bt = static_cast<uint32_t>(i / (static_cast<unsigned long long>(kq) * p.N)); }
        const uint32_t k0 = q * 4;
        float v[4], lo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            v[j] = (k0 + j < p.K) ? p.b[bt * p.b_b + static_cast<long long>(n) * p.b_n + static_cast<long long>(k0 + j) * p.b_k] : 0.0f;
            lo[j] = tf32_low_part(__float_as_uint(v[j]));
        }
        const unsigned long long row = static_cast<unsigned long long>(bt) * p.N + n;
        *reinterpret_cast<float4*>(p.bh + row * p.Kp + k0) = make_float4(v[0], v[1], v[2], v[3]);
        // k-block kb of the row: [ b16(b) x 32 | lo(b) x 32 ]
        const uint32_t kb = k0 / 32, within = k0 % 32;
        __nv_bfloat16* dst = p.bc + row * (2ull * p.Kp) + kb * 64ull + within;
        uint2 hi2, lo2;
        hi2.x = pack2<__nv_bfloat16>(v[0], v[1]); hi2.y = pack2<__nv_bfloat16>(v[2], v[3]);
        lo2.x = pack2<__nv_bfloat16>(lo[0], lo[1]); lo2.y = pack2<__nv_bfloat16>(lo[2], lo[3]);
        *reinterpret_cast<uint2*>(dst) = hi2;
        *reinterpret_cast<uint2*>(dst + 32) = lo2;
    }
}

// Epilogue of this kernel: main + correction accumulators -> bias, activation -> memory, 32 columns (one 128-byte
// segment of 32 rows) at a time.  tcgen05.wait::ld waits for every load of the thread, so the loads of the next
// segment are issued right after the wait for the current one: their latency passes while the current segment is
// staged and stored.  The store paths are those of drain_accumulator.
template <uint32_t BN, uint32_t PARTS>
__device__ __forceinline__ void drain_two_accumulators(const GemmParams& p, const CUtensorMap* tmap_out, uint32_t staging,
                                                       uint32_t part, uint32_t acc, uint32_t acc2, uint32_t quarter,
                                                       uint32_t lane, uint32_t batch, uint32_t m0, uint32_t n0)
{
    constexpr uint32_t kPer = BN / 32 / PARTS;                  // segments per warp
    static_assert(kPer % 2 == 0, "segments are handled in pairs");
    float* const out = static_cast<float*>(p.out);
    const float* const bias = static_cast<const float*>(p.bias);
    const uint32_t row = m0 + quarter * 32 + lane;
    const uint32_t lane_addr = (quarter * 32u) << 16;
    float row_bias = 0.0f;
    if (p.bias_mode == 2 && row < p.M) row_bias = bias[static_cast<long long>(row) * p.bias_stride];
    float* row_ptr = out + static_cast<long long>(batch) * p.out_batch_stride + static_cast<long long>(row) * p.ldo;

    auto load = [&](uint32_t i, uint32_t (&x)[32], uint32_t (&y)[32]) {
        const uint32_t col = (part + i * PARTS) * 32;
        tmem_ld_32x32(acc + lane_addr + col, x);
        tmem_ld_32x32(acc2 + lane_addr + col, y);
    };
    auto finish = [&](uint32_t i, uint32_t (&x)[32], uint32_t (&y)[32]) {
        const uint32_t col0 = n0 + (part + i * PARTS) * 32;
        if (col0 >= p.N) return;                                // uniform over the warp
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(x[j]) + __uint_as_float(y[j]);
        if (p.bias_mode == 1) {
            float my_bias = 0.0f;                               // one coalesced load, handed out by shuffle
            if (col0 + lane < p.N) my_bias = __ldg(bias + static_cast<long long>(col0 + lane) * p.bias_stride);
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += __shfl_sync(0xffffffffu, my_bias, j);
        } else if (p.bias_mode == 2) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += row_bias;
        }
        activate_chunk(p.act, v);
        if (!p.out_tma) {
            if (row < p.M) store_row_chunk<float>(p, row_ptr, col0, v);
            return;
        }
        if (lane == 0) bulk_wait_group_read<0>();               // the previous store has read the staging buffer
        __syncwarp();
#pragma unroll
        for (uint32_t q = 0; q < 8; ++q) {
            const uint32_t addr = staging + lane * 128 + ((q ^ (lane & 7)) << 4);
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};"
                         ::"r"(addr), "r"(__float_as_uint(v[4 * q])), "r"(__float_as_uint(v[4 * q + 1])),
                           "r"(__float_as_uint(v[4 * q + 2])), "r"(__float_as_uint(v[4 * q + 3])) : "memory");
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
            tma_store_3d(tmap_out, staging, static_cast<int32_t>(col0), static_cast<int32_t>(m0 + quarter * 32),
                         static_cast<int32_t>(batch));
            bulk_commit_group();
        }
    };
    uint32_t x0[32], y0[32], x1[32], y1[32];
    load(0, x0, y0);
#pragma unroll
    for (uint32_t i = 0; i < kPer; i += 2) {
        tmem_ld_wait_regs2(x0, y0);
        load(i + 1, x1, y1);
        finish(i, x0, y0);
        tmem_ld_wait_regs2(x1, y1);
        if (i + 2 < kPer) load(i + 2, x0, y0);
        finish(i + 1, x1, y1);
    }
}

struct X3Params {
    GemmParams g;                 // sizes, tile walk, A descriptor fields, epilogue
    uint32_t idesc_tf32, idesc_bf16;
};

template <uint32_t BN>
__global__ void __launch_bounds__(x3_threads(BN), 1)
gemm_tf32x3_pair_kernel(const __grid_constant__ CUtensorMap tmap_a,
                        const __grid_constant__ CUtensorMap tmap_bh,
                        const __grid_constant__ CUtensorMap tmap_bc,
                        const __grid_constant__ CUtensorMap tmap_out,
                        const __grid_constant__ X3Params xp)
{
    const GemmParams& p = xp.g;
    constexpr uint32_t kStageBytes = x3_stage_bytes(BN);
    constexpr uint32_t kStages = x3_stages(BN);
    constexpr uint32_t kBTileBytes = (BN / 2) * kRowBytes;          // this CTA's half of the Bh (or Bc) tile
    constexpr bool kOverlap = BN == 128;                            // separate epilogue warps, double-buffered accumulators
    constexpr uint32_t kAccBufs = kOverlap ? 2 : 1;
    constexpr uint32_t kEpiWarps = x3_epilogue_warps(BN);
    constexpr uint32_t kTmemCols = 512;             // per buffer: main accumulator (BN columns), then corrections (BN columns)

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

    __shared__ __align__(8) uint64_t full_a[kX3MaxStages];       // own A tile landed
    __shared__ __align__(8) uint64_t full_b[kX3MaxStages];       // leader: both CTAs' Bh and Bc tiles landed
    __shared__ __align__(8) uint64_t ready[kX3MaxStages];        // leader: both CTAs' correction tiles written
    __shared__ __align__(8) uint64_t empty_bar[kX3MaxStages];    // both: the stage's MMAs have completed
    __shared__ __align__(8) uint64_t tmem_full_bar[2];
    __shared__ __align__(8) uint64_t tmem_empty_bar[2];          // leader: one arrive per epilogue warp of both CTAs
    __shared__ __align__(8) uint64_t drain_bar;
    __shared__ uint32_t tmem_holder;
    __shared__ volatile uint32_t abort_flag;
    __shared__ volatile uint32_t never_set;          // the drain waits' stand-in for an abort flag
    __shared__ uint32_t issued_loads;               // k-block iterations whose loads this CTA's producer issued

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t cta_rank = cluster_ctarank();
    const uint32_t pair_id = blockIdx.x >> 1;
    const uint32_t num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        never_set = 0;
        issued_loads = 0;
        mbar_init(smem_u32(&drain_bar), 1);
        for (uint32_t s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&full_a[s]), 1);
            mbar_init(smem_u32(&full_b[s]), 1);
            mbar_init(smem_u32(&ready[s]), 2 * kX3TransformWarps);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (uint32_t i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&tmem_full_bar[i]), 1);
            mbar_init(smem_u32(&tmem_empty_bar[i]), 2 * kEpiWarps);
        }
        fence_mbar_init();
        prefetch_tensormap(&tmap_a);
        prefetch_tensormap(&tmap_bh);
        prefetch_tensormap(&tmap_bc);
        if (p.out_tma) prefetch_tensormap(&tmap_out);
    }
    if (warp == 1) {
        tmem_alloc_cta2(smem_u32(&tmem_holder), kTmemCols);
        tmem_relinquish_cta2();
    }
    tc_fence_before_sync();
    cluster_arrive_release();
    cluster_wait_acquire();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_holder;
    // an abort is raised in both CTAs of the pair, so that the partner's waits end at once too
    auto raise_abort = [&](uint32_t code) {
        abort_flag = 1;
        st_shared_remote_u32(smem_u32(const_cast<uint32_t*>(&abort_flag)), cta_rank ^ 1u, 1u);
        atomicOr(&g_gemm_status, code);
    };
    // the loads of this CTA for k-block kb of tile tc into a stage
    auto issue_stage = [&](const TileCoord& tc, uint32_t kb, uint32_t stage) {
        const uint32_t m0 = tc.m0 * 2 + cta_rank * kTileM, n0 = tc.n0 + cta_rank * (BN / 2);
        const uint32_t sa = smem_base + stage * kStageBytes;
        const uint32_t sbh = sa + 2 * kX3TileBytes, sbc = sbh + kBTileBytes;
        const uint32_t bar_a = smem_u32(&full_a[stage]);
        const uint32_t bar_b = map_to_cta(smem_u32(&full_b[stage]), 0);
        mbar_arrive_expect_tx(bar_a, kX3TileBytes);
        if (cta_rank == 0) mbar_arrive_expect_tx(smem_u32(&full_b[stage]), 4 * kBTileBytes);
        tma_load_3d(sa, &tmap_a, bar_a, static_cast<int32_t>(kb * 32), m0, tc.batch * p.a.batch_mul);
        tma_load_3d_pair(sbh, &tmap_bh, bar_b, static_cast<int32_t>(kb * 32), n0, tc.batch * p.b.batch_mul);
        tma_load_3d_pair(sbc, &tmap_bc, bar_b, static_cast<int32_t>(kb * 64), n0, tc.batch * p.b.batch_mul);
    };
    // the same for k-block iteration j of the pair's work list (every tile has p.k_blocks of them): the teardown's form
    auto issue_loads = [&](uint32_t j) {
        const uint32_t t_local = j / p.k_blocks;
        issue_stage(decode_tile(p, pair_id + t_local * num_pairs, BN), j - t_local * p.k_blocks, j % kStages);
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        if (elect_one()) {
            uint32_t stage = 0, phase = 0, issued = 0;
            bool ok = true;
            grid_dependency_wait();                  // Bh / Bc come from the pack kernel launched just before
            for (uint32_t tile = pair_id; ok && tile < p.num_tiles; tile += num_pairs) {
                const TileCoord tc = decode_tile(p, tile, BN);       // once per tile: nothing is divided between a freed stage and its loads
                for (uint32_t kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait_cluster(smem_u32(&empty_bar[stage]), phase ^ 1, &abort_flag, p.wait_cycles)) { ok = false; break; }
                    issue_stage(tc, kb, stage);
                    ++issued;
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
            }
            issued_loads = issued;
            if (!ok) raise_abort(kStatusProducerTimeout);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (leader CTA)
        if (cta_rank == 0 && elect_one()) {
            uint32_t stage = 0, phase = 0, local = 0;
            bool ok = true;
            const uint64_t hi64 = static_cast<uint64_t>(p.a.desc_hi) << 32;     // K-major, 128-byte swizzle: every tile alike
            for (uint32_t tile = pair_id; ok && tile < p.num_tiles; tile += num_pairs, ++local) {
                const uint32_t buf = local % kAccBufs, acc_phase = (local / kAccBufs) & 1;
                if (!mbar_wait_cluster(smem_u32(&tmem_empty_bar[buf]), acc_phase ^ 1, &abort_flag, p.wait_cycles)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t d_main = tmem_base + buf * 2 * BN, d_corr = d_main + BN;
                for (uint32_t kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait_cluster(smem_u32(&full_b[stage]), phase, &abort_flag, p.wait_cycles)) { ok = false; break; }
                    if (!mbar_wait_cluster(smem_u32(&ready[stage]), phase, &abort_flag, p.wait_cycles)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t sa = smem_base + stage * kStageBytes;
                    const uint32_t a_raw = ((sa >> 4) & 0x3fffu) | p.a.desc_lo_fixed;
                    const uint32_t a_cor = (((sa + kX3TileBytes) >> 4) & 0x3fffu) | p.a.desc_lo_fixed;
                    const uint32_t b_raw = (((sa + 2 * kX3TileBytes) >> 4) & 0x3fffu) | p.a.desc_lo_fixed;
                    const uint32_t b_cor = (((sa + 2 * kX3TileBytes + kBTileBytes) >> 4) & 0x3fffu) | p.a.desc_lo_fixed;
                    const uint32_t first = (kb != 0);
#pragma unroll
                    for (uint32_t k = 0; k < 4; ++k)          // 32 fp32 of K: four TF32 MMAs of K = 8 (32 bytes each)
                        umma_tf32_cta2(d_main, hi64 | (a_raw + k * 2), hi64 | (b_raw + k * 2), xp.idesc_tf32, first | k);
#pragma unroll
                    for (uint32_t k = 0; k < 4; ++k)          // 64 bf16 of K: four BFloat16 MMAs of K = 16 (32 bytes each)
                        umma_f16_cta2(d_corr, hi64 | (a_cor + k * 2), hi64 | (b_cor + k * 2), xp.idesc_bf16, first | k);
                    umma_commit_cta2_mc(smem_u32(&empty_bar[stage]), 3);
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
                if (ok) umma_commit_cta2_mc(smem_u32(&tmem_full_bar[buf]), 3);
            }
            if (!ok) raise_abort(kStatusMmaTimeout);
        }
    } else {
        // ------------------------------------------------------------------ transform and epilogue (both CTAs)
        // BN = 256: warps 2-9 do both, one after the other (the accumulators fill TMEM, so there is nothing to
        // overlap).  BN = 128: warps 2-5 are the epilogue, warps 6-13 the transform, each in its own loop.
        const bool transforms = !kOverlap || warp >= 2 + kEpiWarps;
        const bool drains = !kOverlap || warp < 2 + kEpiWarps;
        const uint32_t wt = threadIdx.x - (kOverlap ? (2 + kEpiWarps) * 32 : 64);      // 0 .. 255 among the transform threads
        const uint32_t row = wt & 127, half = wt >> 7;          // half a row of the A tile: 16 of its 32 values
        const uint32_t sw = row & 7;
        const uint32_t quarter = warp & 3;
        uint32_t stage = 0, phase = 0, local = 0;
        bool ok = true;
        for (uint32_t tile = pair_id; ok && tile < p.num_tiles; tile += num_pairs, ++local) {
            const TileCoord tc = decode_tile(p, tile, BN);
            if (transforms) {
                for (uint32_t kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait(smem_u32(&full_a[stage]), phase, &abort_flag, p.wait_cycles)) { ok = false; break; }
                    const uint32_t src = smem_base + stage * kStageBytes + row * 128;
                    const uint32_t dst = src + kX3TileBytes;
                    uint32_t x[16];
#pragma unroll
                    for (uint32_t c = 0; c < 4; ++c)                 // logical 16-byte chunks 4 half .. 4 half + 3 of the row
                        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                                     : "=r"(x[4 * c]), "=r"(x[4 * c + 1]), "=r"(x[4 * c + 2]), "=r"(x[4 * c + 3])
                                     : "r"(src + (((4 * half + c) ^ sw) << 4)));
                    uint32_t lo[8], hi[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        lo[e] = pack2<__nv_bfloat16>(tf32_low_part(x[2 * e]), tf32_low_part(x[2 * e + 1]));
                        hi[e] = pack2<__nv_bfloat16>(__uint_as_float(x[2 * e]), __uint_as_float(x[2 * e + 1]));
                    }
#pragma unroll
                    for (uint32_t c = 0; c < 2; ++c) {               // 8 values each: chunk 2 half + c of lo, chunk 4 + 2 half + c of b16
                        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};"
                                     ::"r"(dst + (((2 * half + c) ^ sw) << 4)), "r"(lo[4 * c]), "r"(lo[4 * c + 1]), "r"(lo[4 * c + 2]),
                                       "r"(lo[4 * c + 3]) : "memory");
                        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};"
                                     ::"r"(dst + (((4 + 2 * half + c) ^ sw) << 4)), "r"(hi[4 * c]), "r"(hi[4 * c + 1]), "r"(hi[4 * c + 2]),
                                       "r"(hi[4 * c + 3]) : "memory");
                    }
                    fence_proxy_async_smem();          // generic-proxy writes -> visible to the MMA's reads
                    __syncwarp();
                    if (lane == 0) mbar_arrive_remote(smem_u32(&ready[stage]), 0);
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
            }
            if (drains) {
                const uint32_t buf = local % kAccBufs, acc_phase = (local / kAccBufs) & 1;
                const uint32_t m0 = tc.m0 * 2 + cta_rank * kTileM;
                if (!mbar_wait_cluster(smem_u32(&tmem_full_bar[buf]), acc_phase, &abort_flag, p.wait_cycles)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t acc = tmem_base + buf * 2 * BN;
                drain_two_accumulators<BN, kEpiWarps / 4>(p, &tmap_out, smem_base + kStages * kStageBytes + (warp - 2) * 4096,
                                                          (warp - 2) >> 2, acc, acc + BN, quarter, lane, tc.obatch, m0, tc.n0);
                tc_fence_before_sync();
                __syncwarp();
                // the accumulator reads have completed (tcgen05.wait::ld) and nothing in memory is handed over: the
                // plain arrive is enough, and unlike the cluster-scope release it does not wait for this warp's stores
                if (lane == 0) mbar_arrive_remote(smem_u32(&tmem_empty_bar[buf]), 0);
            }
        }
        if (drains) drain_finish(lane);
        if (!ok && lane == 0) raise_abort(drains ? kStatusEpilogueTimeout : kStatusPairTimeout);
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncwarp();
    cluster_arrive_release();
    cluster_wait_acquire();
    if (abort_flag != 0) {
        // As in gemm_tcgen05_pair_kernel: the leader waits for the MMAs issued so far, the producer that is
        // behind issues the loads its partner already issued, then every producer waits for its own A stages
        // and the leader for the stages of the packed operand.
        if (cta_rank == 0 && warp == 1 && lane == 0) {
            umma_commit_cta2_mc(smem_u32(&drain_bar), 1);
            mbar_wait_cluster(smem_u32(&drain_bar), 0, &never_set, kDrainCycles);
        }
        __syncwarp();
        cluster_arrive_release();
        cluster_wait_acquire();
        uint32_t both = 0;
        if (warp == 0 && lane == 0) {
            const uint32_t mine = issued_loads, theirs = ld_shared_remote_u32(smem_u32(&issued_loads), cta_rank ^ 1u);
            for (uint32_t j = mine; j < theirs; ++j) issue_loads(j);
            both = mine > theirs ? mine : theirs;
        }
        __syncwarp();
        cluster_arrive_release();
        cluster_wait_acquire();
        if (warp == 0 && lane == 0) {
            drain_armed_stages(full_a, kStages, both, &never_set);
            if (cta_rank == 0) drain_armed_stages(full_b, kStages, both, &never_set);
        }
        __syncwarp();
        cluster_arrive_release();
        cluster_wait_acquire();
    }
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_cta2(tmem_base, kTmemCols);
    }
    cluster_arrive_release();
    cluster_wait_acquire();
}

}  // namespace srt
