// Tensor-core GEMM for sm_100a: one CTA per 128 x BN output tile, persistent over tiles.
//
//   warp 0      TMA producer: fills a ring of shared-memory stages (A tile + B tile, 128-byte
//               swizzled rows) with cp.async.bulk.tensor loads, one mbarrier per stage.
//   warp 1      MMA issuer: one thread issues tcgen05.mma (128 x BN x 32 bytes of K per
//               instruction) from the shared-memory descriptors into a TMEM accumulator;
//               tcgen05.commit hands each stage back to the producer and each finished
//               accumulator to the epilogue.  Also owns the TMEM allocation.
//   warps 2-9   epilogue: tcgen05.ld the fp32 accumulator (warp w reads TMEM lanes 32 (w mod 4) ..,
//               two warps per lane quarter taking alternate 128-byte column segments), add bias,
//               apply the activation, round once to the output type, store.
//
// The accumulator is double-buffered in TMEM (2 x BN columns), so the epilogue of tile i
// overlaps the main loop of tile i + 1.  Operands may be K-major (K contiguous) or
// MN-major (M or N contiguous); the difference is confined to the TMA box shapes and the
// descriptor fields the host prepares in GemmParams.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ptx.cuh"

namespace srt {

constexpr uint32_t kTileM = 128;        // rows of one MMA (all 128 TMEM lanes)
constexpr uint32_t kRowBytes = 128;     // swizzle span = bytes of one shared-memory tile row
constexpr uint32_t kATileBytes = kTileM * kRowBytes;
constexpr uint32_t kKStepsPerStage = 4; // MMAs per stage: each consumes 32 bytes of K
constexpr uint32_t kGemmThreads = 320;      // producer warp, MMA warp, 8 epilogue warps

enum : uint32_t {
    kStatusProducerTimeout = 1u,
    kStatusMmaTimeout = 2u,
    kStatusEpilogueTimeout = 4u,
    kStatusPairTimeout = 8u
};

// Status word of the tensor-core kernels, one per device that loads the module.
__device__ uint32_t g_gemm_status;

struct OperandParams {
    uint32_t mn_major;      // 0: K contiguous, 1: M/N contiguous
    uint32_t chunks;        // TMA boxes per stage (1 for K-major)
    uint32_t chunk_elems;   // M/N elements per box (MN-major)
    uint32_t chunk_bytes;   // shared-memory bytes per box
    uint32_t batch_mul;     // 0 broadcasts the operand over the batch
    uint32_t desc_hi;       // upper half of the shared-memory matrix descriptor
    uint32_t desc_lo_fixed; // leading-byte-offset field, already shifted
    uint32_t kstep;         // descriptor start-address increment per MMA (bytes >> 4)
};

// Division of a number below 2^31 by a divisor fixed on the host: floor(n / d) = umulhi(n, mul) >> shr with
// mul = ceil(2^(31 + ceil(log2 d)) / d) (Granlund-Montgomery); d = 1 is passed through.  The tile walk divides by
// five such numbers per tile, and a 32-bit hardware-less division is some thirty dependent instructions: about
// 600 cycles per tile on each role's path, which is most of what a tile costs when it has one or two k-blocks.
struct FastDiv {
    uint32_t mul, shr, d;
};

inline FastDiv make_fast_div(uint32_t d)
{
    FastDiv f = {0u, 0u, d == 0 ? 1u : d};
    if (f.d == 1) return f;
    uint32_t lg = 0;
    while ((1ull << lg) < f.d) ++lg;                       // ceil(log2 d)
    const uint32_t pw = 31 + lg;
    f.mul = static_cast<uint32_t>(((1ull << pw) + f.d - 1) / f.d);
    f.shr = pw - 32;
    return f;
}

__device__ __forceinline__ uint32_t fast_div(uint32_t n, const FastDiv& f)
{
    return f.d == 1 ? n : (__umulhi(n, f.mul) >> f.shr);
}

struct GemmParams {
    uint32_t M, N, K, batch;
    uint32_t tiles_m, tiles_n, tiles_per_batch, num_tiles;
    uint32_t k_blocks, kb_elems, group_m;
    uint32_t k_splits, kb_per_split;   // split-K: work unit = (tile, split); num_tiles counts units
    uint32_t tiles_total;              // output tiles over all batch items (= num_tiles / k_splits)
    FastDiv by_tiles_total, by_tiles_per_batch, by_per_group, by_group_m, by_group_tail;   // set_tile_walk()
    OperandParams a, b;
    uint32_t idesc;
    uint32_t stage_tx_bytes;
    uint32_t stages;
    // epilogue
    void* out;
    long long ldo;               // elements between output rows (columns are contiguous)
    long long out_batch_stride;  // elements
    const void* bias;
    long long bias_stride;
    uint32_t bias_mode;          // 0 none, 1 one value per column, 2 one value per row
    uint32_t act;
    uint32_t out_vec_ok;         // 16-byte vector stores are aligned for every full chunk
    uint32_t out_tma;            // the output view is TMA-addressable: bulk tensor stores from shared memory
    uint32_t n_peers;            // gathering kernels only: peer copies of the output view (<= kMaxPeers)
    uint32_t multicast;          // gathering kernels only: 1 = the result goes to a multicast mapping instead (no per-peer stores)
    unsigned long long wait_cycles;   // limit of every pipeline wait, in SM clock cycles (set at launch)
    // LSTM epilogue (epilogue == kEpilogueLstm): the product's columns are the interleaved gate pre-activations
    // (4 j + g for gate g of hidden unit j); nothing of the product is stored, the new cell and hidden states are
    uint32_t epilogue;           // 0: bias / activation / store; 1: LSTM gates
    const void* lstm_cell; void* lstm_new_cell; void* lstm_new_hidden;
    long long lstm_c_m, lstm_nc_m, lstm_nh_m;   // row strides in elements (columns are contiguous)
};

enum : uint32_t { kEpilogueStore = 0, kEpilogueLstm = 1 };
enum : uint32_t { kActSigmoid = 0, kActRelu = 1, kActTanh = 2, kActIdentity = 5, kActGelu = 6, kActGeluTanh = 7 };

__device__ __forceinline__ float apply_activation(uint32_t act, float x)
{
    switch (act) {
    case kActRelu: return x >= 0.0f ? x : 0.0f;
    case kActSigmoid: return 1.0f / (1.0f + expf(-x));
    case kActTanh: return tanhf(x);
    case kActGelu: return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
    case kActGeluTanh: {
        float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
        return 0.5f * x * (1.0f + tanhf(u));
    }
    default: return x;
    }
}

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi)
{
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi)
{
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Low part of an fp32 value for the split-precision kernels: x - hi(x), where hi(x) is x with its low
// 13 mantissa bits cleared (what a TF32 MMA reads from the word).  Two exceptions keep non-finite
// inputs on the reference's results: an infinity or NaN is its own low part (so that every term it
// enters carries it), and a zero low part of a non-zero value is replaced by x 2^-30 -- far below the
// lo . lo term these kernels drop -- so that infinity times such a value stays an infinity instead of
// inf . 0 = NaN.  (Values below 2^-96 still lose that tiny stand-in to underflow.)
__device__ __forceinline__ float tf32_low_part(uint32_t x)
{
    const float v = __uint_as_float(x);
    const float lo = v - __uint_as_float(x & 0xffffe000u);
    // |lo| > 0 is false for a zero low part and for the NaN that inf - inf or NaN - NaN gives, and v 2^-30 is then
    // the stand-in of a finite v, and v itself for an infinity or a NaN: one ordered comparison covers all cases
    return fabsf(lo) > 0.0f ? lo : v * 9.31322574615478515625e-10f;          // 2^-30
}

// work unit -> tile coordinates; m-tiles are visited in groups of group_m so that the CTAs running
// at the same time share A and B tiles in L2.  With split-K, unit u is split u / tiles_total of
// tile u % tiles_total: it reduces k-blocks [kb0, kb1) and writes partial sums to the slice
// `obatch` of an fp32 workspace laid out [split][batch][M][N].
struct TileCoord {
    uint32_t batch, obatch, m0, n0, kb0, kb1;
};

// the divisors of decode_tile, from the tile counts (host side, after tiles_m, tiles_n, tiles_per_batch, tiles_total
// and group_m are set)
inline void set_tile_walk(GemmParams& p)
{
    p.by_tiles_total = make_fast_div(p.tiles_total);
    p.by_tiles_per_batch = make_fast_div(p.tiles_per_batch);
    p.by_per_group = make_fast_div(p.group_m * p.tiles_n);
    p.by_group_m = make_fast_div(p.group_m);
    p.by_group_tail = make_fast_div(p.tiles_m % p.group_m);
}

__device__ __forceinline__ TileCoord decode_tile(const GemmParams& p, uint32_t unit, uint32_t bn)
{
    TileCoord c;
    const uint32_t split = fast_div(unit, p.by_tiles_total);
    const uint32_t tile = unit - split * p.tiles_total;
    c.batch = fast_div(tile, p.by_tiles_per_batch);
    uint32_t t = tile - c.batch * p.tiles_per_batch;
    uint32_t per_group = p.group_m * p.tiles_n;
    uint32_t group = fast_div(t, p.by_per_group);
    uint32_t first_m = group * p.group_m;
    uint32_t gm = min(p.group_m, p.tiles_m - first_m);      // group_m, or what is left of the rows in the last group
    uint32_t r = t - group * per_group;
    const uint32_t col = fast_div(r, gm == p.group_m ? p.by_group_m : p.by_group_tail);
    c.m0 = (first_m + (r - col * gm)) * kTileM;
    c.n0 = col * bn;
    c.obatch = split * p.batch + c.batch;
    c.kb0 = split * p.kb_per_split;
    c.kb1 = min(p.k_blocks, c.kb0 + p.kb_per_split);
    return c;
}

// Stores 32 consecutive columns of one output row held as fp32 in v[].
template <typename OutT>
__device__ __forceinline__ void store_row_chunk(const GemmParams& p, OutT* row_ptr, uint32_t col0,
                                                const float (&v)[32])
{
    if (p.out_vec_ok && col0 + 32 <= p.N) {
        if constexpr (sizeof(OutT) == 4) {
            float4* dst = reinterpret_cast<float4*>(row_ptr + col0);
#pragma unroll
            for (int j = 0; j < 8; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        } else {
            uint4* dst = reinterpret_cast<uint4*>(row_ptr + col0);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint4 q;
                q.x = pack2<OutT>(v[8 * j + 0], v[8 * j + 1]);
                q.y = pack2<OutT>(v[8 * j + 2], v[8 * j + 3]);
                q.z = pack2<OutT>(v[8 * j + 4], v[8 * j + 5]);
                q.w = pack2<OutT>(v[8 * j + 6], v[8 * j + 7]);
                dst[j] = q;
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) row_ptr[col0 + j] = from_float<OutT>(v[j]);
    }
}

// Applies the activation to a chunk of 32 values; the selector is uniform, so the switch is
// taken once per chunk and each case is a straight loop.
__device__ __forceinline__ void activate_chunk(uint32_t act, float (&v)[32])
{
    switch (act) {
    case kActIdentity: break;
    case kActRelu:
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = v[j] >= 0.0f ? v[j] : 0.0f;
        break;
    case kActSigmoid:
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = apply_activation(kActSigmoid, v[j]);
        break;
    case kActTanh:
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = apply_activation(kActTanh, v[j]);
        break;
    case kActGelu:
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = apply_activation(kActGelu, v[j]);
        break;
    case kActGeluTanh:
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = apply_activation(kActGeluTanh, v[j]);
        break;
    default: break;
    }
}

// Drains one finished 128-row accumulator (this warp's 32 TMEM lanes, BN columns starting at
// TMEM address `acc`) to global memory: bias, activation, one rounding, stores.
// With DUAL the tile's value is the sum of two accumulators (`acc` and `acc2`), added in fp32.
//
// Two store paths.  When the output view is TMA-addressable (p.out_tma) each warp stages 128-byte
// wide row segments of its 32 rows in shared memory (128-byte swizzle, one 4 KB buffer per warp)
// and one lane issues a bulk tensor store per segment: full-line writes, clipped at the tensor's
// edges by the hardware.  Otherwise every thread stores its own row with 16-byte or scalar stores.
constexpr uint32_t kEpilogueStagingBytes = 8 * 4096;         // 8 warps x (32 rows x 128 B)

// PARTS: how many warps share one lane quarter (1 or 2); warp `part` drains every PARTS-th
// 128-byte column segment.  `staging` is this warp's own 4 KB buffer.
//
// GATHER: every staged segment is also stored through the tensor maps of `peers` (the same view
// in the output buffers of other GPUs, mapped into this process), so that all of them hold the
// tile when the kernel has finished.  Bulk tensor STORES to peer memory only; nothing is loaded
// from a peer and no peer is waited for.  With p.multicast the segment is instead read back from
// the staging buffer and stored once, 16 bytes per lane, to a multicast mapping of the view
// (multimem.st): the NVSwitch replicates it to every GPU, this one included, so each byte leaves
// the GPU once instead of once per peer.
constexpr uint32_t kMaxPeers = 7;
struct PeerMaps { CUtensorMap m[kMaxPeers]; void* multicast; };
struct NoPeers { uint32_t unused; };
template <bool GATHER> struct PeerArgOf { using type = NoPeers; };
template <> struct PeerArgOf<true> { using type = PeerMaps; };

// `rehearsal` (drain_accumulator): run the whole epilogue once on whatever an idle accumulator buffer holds, with
// every store left out.  The epilogue warps have nothing to do while the first tile is reduced, and the first
// execution of the epilogue on an SM otherwise waits for its instructions to arrive (about 4000 cycles on the first
// 32-row segment after another kernel has run there, against 1600-1900 for the following ones): rehearsed under the
// reduction, the real epilogue runs from a warm instruction cache.  Only worth it where the epilogue is exposed.
//
// The bias values one epilogue warp needs for one tile: per 32-column chunk it drains, the value of this lane's
// column (handed out to the other lanes by shuffle), or the value of this thread's row.  They are loaded BEFORE the
// warp waits for the tile's accumulator, so that their latency (a trip to HBM when the cache is cold) passes under
// the reduction instead of inside the epilogue: on a single-wave Dense product the epilogue is exposed in full.
template <typename T, uint32_t BN, uint32_t PARTS>
struct TileBias {
    static constexpr uint32_t kColsPerBox = 128 / sizeof(T), kLoadsPerBox = kColsPerBox / 32, kBoxes = BN / kColsPerBox;
    static constexpr uint32_t kChunks = ((kBoxes + PARTS - 1) / PARTS) * kLoadsPerBox;
    float col[kChunks];
    float row;
};

template <typename T, uint32_t BN, uint32_t PARTS>
__device__ __forceinline__ void load_tile_bias(const GemmParams& p, uint32_t part, uint32_t quarter, uint32_t lane, uint32_t m0,
                                               uint32_t n0, TileBias<T, BN, PARTS>& tb)
{
    using TB = TileBias<T, BN, PARTS>;
    const T* const bias = static_cast<const T*>(p.bias);
    tb.row = 0.0f;
#pragma unroll
    for (uint32_t c = 0; c < TB::kChunks; ++c) tb.col[c] = 0.0f;
    if (p.bias_mode == 0) return;
    const uint32_t row = m0 + quarter * 32 + lane;
    if (p.bias_mode == 2 && row < p.M) tb.row = to_float<T>(__ldg(bias + static_cast<long long>(row) * p.bias_stride));
#pragma unroll
    for (uint32_t c = 0; c < TB::kChunks; ++c) {
        const uint32_t bx = part + (c / TB::kLoadsPerBox) * PARTS;
        const uint32_t col = n0 + bx * TB::kColsPerBox + (c % TB::kLoadsPerBox) * 32 + lane;
        if (p.bias_mode == 1 && bx < TB::kBoxes && col < p.N) tb.col[c] = to_float<T>(__ldg(bias + static_cast<long long>(col) * p.bias_stride));
    }
}

template <typename T, uint32_t BN, bool DUAL = false, uint32_t PARTS = 1, bool GATHER = false>
__device__ __forceinline__ void drain_accumulator(const GemmParams& p, const CUtensorMap* tmap_out, uint32_t staging,
                                                  uint32_t part, uint32_t acc, uint32_t quarter, uint32_t lane,
                                                  uint32_t batch, uint32_t m0, uint32_t n0, TileBias<T, BN, PARTS> tb,
                                                  uint32_t acc2 = 0, const PeerMaps* peers = nullptr, uint32_t rehearsal = 0)
{
    constexpr uint32_t kColsPerBox = 128 / sizeof(T);            // 64 (16-bit) or 32 (fp32)
    constexpr uint32_t kLoadsPerBox = kColsPerBox / 32;
    constexpr uint32_t kBoxes = BN / kColsPerBox;
    T* const out = static_cast<T*>(p.out);
    const uint32_t row = m0 + quarter * 32 + lane;
    const uint32_t lane_addr = (quarter * 32u) << 16;
    const float row_bias = tb.row;
    T* row_ptr = out + static_cast<long long>(batch) * p.out_batch_stride + static_cast<long long>(row) * p.ldo;

    for (uint32_t bx = part; bx < kBoxes; bx += PARTS) {
        const uint32_t box_col = n0 + bx * kColsPerBox;
        if (box_col >= p.N) break;                              // uniform over the warp
        uint32_t packed[32];                                    // 128 bytes of this thread's output row
        // all accumulator loads of the box are issued before the first wait: their latencies overlap
        uint32_t raw[kLoadsPerBox][32];
#pragma unroll
        for (uint32_t h = 0; h < kLoadsPerBox; ++h) tmem_ld_32x32(acc + lane_addr + (bx * kLoadsPerBox + h) * 32, raw[h]);
#pragma unroll
        for (uint32_t h = 0; h < kLoadsPerBox; ++h) {
            const uint32_t col0 = box_col + h * 32;
            const float my_bias = tb.col[h];      // this lane's column of the chunk, handed out by shuffle below
            if (h == 0) {
                if constexpr (kLoadsPerBox == 2) tmem_ld_wait_regs2(raw[0], raw[kLoadsPerBox - 1]);
                else tmem_ld_wait_regs(raw[0]);
            }
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[h][j]);
            if constexpr (DUAL) {
                uint32_t raw2[32];
                tmem_ld_32x32(acc2 + lane_addr + (bx * kLoadsPerBox + h) * 32, raw2);
                tmem_ld_wait_regs(raw2);
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] += __uint_as_float(raw2[j]);
            }
            if (p.bias_mode == 1) {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] += __shfl_sync(0xffffffffu, my_bias, j);
            } else if (p.bias_mode == 2) {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] += row_bias;
            }
            activate_chunk(p.act, v);
            if (!p.out_tma) {
                if (row < p.M && col0 < p.N && !rehearsal) store_row_chunk<T>(p, row_ptr, col0, v);
            } else if constexpr (sizeof(T) == 4) {
#pragma unroll
                for (int j = 0; j < 32; ++j) packed[j] = __float_as_uint(v[j]);
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) packed[h * 16 + j] = pack2<T>(v[2 * j], v[2 * j + 1]);
            }
        }
        if (p.out_tma) {
            // the previous store of this warp read the same buffer: it must have finished reading
            if (lane == 0) bulk_wait_group_read<0>();
            __syncwarp();
#pragma unroll
            for (uint32_t q = 0; q < 8; ++q) {
                const uint32_t addr = staging + lane * 128 + ((q ^ (lane & 7)) << 4);
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};"
                             ::"r"(addr), "r"(packed[4 * q]), "r"(packed[4 * q + 1]), "r"(packed[4 * q + 2]),
                               "r"(packed[4 * q + 3]) : "memory");
            }
            fence_proxy_async_smem();
            __syncwarp();
            bool multicast = false;
            if constexpr (GATHER) multicast = p.multicast != 0;
            if (rehearsal) {
                __syncwarp();
            } else if (!multicast) {
                if (lane == 0) {
                    tma_store_3d(tmap_out, staging, static_cast<int32_t>(box_col), static_cast<int32_t>(m0 + quarter * 32),
                                 static_cast<int32_t>(batch));
                    if constexpr (GATHER) {
                        for (uint32_t i = 0; i < p.n_peers; ++i)
                            tma_store_3d(&peers->m[i], staging, static_cast<int32_t>(box_col),
                                         static_cast<int32_t>(m0 + quarter * 32), static_cast<int32_t>(batch));
                    }
                    bulk_commit_group();
                }
            } else if constexpr (GATHER) {
                // 8 lanes cover one row of the segment (a full 128-byte line), a warp instruction 4 rows;
                // N is a multiple of 16 bytes here, so a chunk is inside the row or outside it
                constexpr uint32_t kPerChunk = 16 / sizeof(T);
                const uint32_t sub = lane >> 3, q = lane & 7;
                T* const mc = static_cast<T*>(peers->multicast);
#pragma unroll 2
                for (uint32_t it = 0; it < 8; ++it) {
                    const uint32_t r = it * 4 + sub;
                    uint4 v;
                    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                                 : "r"(staging + r * 128 + ((q ^ (r & 7)) << 4)) : "memory");
                    const uint32_t grow = m0 + quarter * 32 + r, gcol = box_col + q * kPerChunk;
                    if (grow < p.M && gcol < p.N)
                        multimem_st_16(mc + static_cast<long long>(batch) * p.out_batch_stride +
                                            static_cast<long long>(grow) * p.ldo + gcol, v);
                }
                __syncwarp();          // every lane has read the segment before the next one is staged
            }
        }
        // the next box's bias values move to the front (static indices: the array stays in registers)
#pragma unroll
        for (uint32_t c = 0; c + kLoadsPerBox < TileBias<T, BN, PARTS>::kChunks; ++c) tb.col[c] = tb.col[c + kLoadsPerBox];
    }
}

// LSTM form of the epilogue.  The weight's columns were interleaved so that the four gate pre-activations of
// hidden unit j -- input, update, forget, output (Part, Sources/SwiftRTLayers/Recurrent.swift:173) -- are columns
// 4 j .. 4 j + 3 of the product: a thread's 32 accumulator columns are 8 whole hidden units.  Per unit
//     cell' = cell * sigmoid(f) + sigmoid(i) * tanh(u),   hidden' = tanh(cell') * sigmoid(o)
// (Recurrent.swift:255-266) in fp32 on the unrounded pre-activations, cell' rounded to the element type before
// hidden' is computed from it.  The thread reads 8 cell values (16 bytes) and writes 8 + 8 (one full 32-byte
// sector per pair of loads): no staging, the fused product itself never reaches memory.
// 16-bit element types; hidden size a multiple of 8; state rows 16-byte aligned.
template <typename T, uint32_t BN, uint32_t PARTS>
__device__ __forceinline__ void drain_accumulator_lstm(const GemmParams& p, uint32_t part, uint32_t acc, uint32_t quarter,
                                                       uint32_t lane, uint32_t m0, uint32_t n0)
{
    static_assert(sizeof(T) == 2, "16-bit element types");
    constexpr uint32_t kBoxes = BN / 64;
    const T* const bias = static_cast<const T*>(p.bias);
    const uint32_t row = m0 + quarter * 32 + lane;
    const uint32_t lane_addr = (quarter * 32u) << 16;
    for (uint32_t bx = part; bx < kBoxes; bx += PARTS) {
        const uint32_t box_col = n0 + bx * 64;
        if (box_col >= p.N) break;                              // uniform over the warp
        uint32_t raw[2][32];
        tmem_ld_32x32(acc + lane_addr + bx * 64, raw[0]);
        tmem_ld_32x32(acc + lane_addr + bx * 64 + 32, raw[1]);
#pragma unroll
        for (uint32_t h = 0; h < 2; ++h) {
            const uint32_t col0 = box_col + h * 32;
            float my_bias = 0.0f;
            if (p.bias_mode == 1 && col0 + lane < p.N)
                my_bias = to_float<T>(__ldg(bias + static_cast<long long>(col0 + lane) * p.bias_stride));
            const uint32_t unit0 = col0 >> 2;
            const bool live = row < p.M && col0 < p.N;
            __align__(16) T c[8];
            if (live) *reinterpret_cast<uint4*>(c) = *reinterpret_cast<const uint4*>(static_cast<const T*>(p.lstm_cell) + static_cast<long long>(row) * p.lstm_c_m + unit0);
            if (h == 0) tmem_ld_wait_regs2(raw[0], raw[1]);
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[h][j]);
            if (p.bias_mode == 1) {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] += __shfl_sync(0xffffffffu, my_bias, j);
            }
            __align__(16) T nc[8], nh[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const float gi = __fdividef(1.0f, 1.0f + __expf(-v[4 * u]));
                const float gu = 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * v[4 * u + 1]));
                const float gf = __fdividef(1.0f, 1.0f + __expf(-v[4 * u + 2]));
                const float go = __fdividef(1.0f, 1.0f + __expf(-v[4 * u + 3]));
                nc[u] = from_float<T>(__fadd_rn(__fmul_rn(to_float<T>(c[u]), gf), __fmul_rn(gi, gu)));
                const float tc = 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * to_float<T>(nc[u])));
                nh[u] = from_float<T>(__fmul_rn(tc, go));
            }
            if (live) {
                *reinterpret_cast<uint4*>(static_cast<T*>(p.lstm_new_cell) + static_cast<long long>(row) * p.lstm_nc_m + unit0) = *reinterpret_cast<const uint4*>(nc);
                *reinterpret_cast<uint4*>(static_cast<T*>(p.lstm_new_hidden) + static_cast<long long>(row) * p.lstm_nh_m + unit0) = *reinterpret_cast<const uint4*>(nh);
            }
        }
    }
}

// Before a warp leaves the kernel (or shared memory is reused for something else) its lane 0
// waits for all its bulk stores.
__device__ __forceinline__ void drain_finish(uint32_t lane)
{
    if (lane == 0) bulk_wait_group<0>();
    __syncwarp();
}

// Orderly end of a kernel in which a wait gave up (abort_flag set).  Before TMEM is released and the CTA
// leaves, nothing asynchronous may still target it: the producer waits for every stage it armed (its
// TMA bytes land whether or not anybody consumes them) and the MMA issuer commits to a barrier of its own
// and waits for it (all MMAs issued so far have then read shared memory and written TMEM).  These waits
// ignore the abort flag and use a limit of their own; on a healthy GPU they last microseconds.
constexpr uint64_t kDrainCycles = 4000000000ull;

__device__ __forceinline__ void drain_armed_stages(uint64_t* full_bar, uint32_t stages, uint32_t issued, volatile uint32_t* never)
{
    for (uint32_t s = 0; s < stages && s < issued; ++s) {
        const uint32_t last = issued - 1 - ((issued - 1 - s) % stages);      // last k-block iteration that used stage s
        mbar_wait(smem_u32(&full_bar[s]), (last / stages) & 1, never, kDrainCycles);
    }
}

// InT / OutT: element type of the inputs and of the output (float, __half, __nv_bfloat16).
// BN: tile width (64, 128 or 256).  fp32 inputs are multiplied as TF32.
// OutT differs from T only for split-K partial sums (16-bit inputs, fp32 workspace).
// GATHER: the epilogue also delivers every tile to the peers (see drain_accumulator).
template <typename T, uint32_t BN, typename OutT = T, bool GATHER = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                    const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_out,
                    const __grid_constant__ GemmParams p,
                    const __grid_constant__ typename PeerArgOf<GATHER>::type peer_maps)
{
    constexpr uint32_t kBTileBytes = BN * kRowBytes;
    constexpr uint32_t kStageBytes = kATileBytes + kBTileBytes;
    constexpr uint32_t kTmemCols = 2 * BN;
    constexpr uint32_t kMaxStages = 8;

    extern __shared__ uint8_t smem_raw[];
    // tiles need 1024-byte alignment for the 128-byte swizzle pattern
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

    __shared__ __align__(8) uint64_t full_bar[kMaxStages];
    __shared__ __align__(8) uint64_t empty_bar[kMaxStages];
    __shared__ __align__(8) uint64_t tmem_full_bar[2];
    __shared__ __align__(8) uint64_t tmem_empty_bar[2];
    __shared__ __align__(8) uint64_t drain_bar;
    __shared__ uint32_t tmem_holder;
    __shared__ volatile uint32_t abort_flag;
    __shared__ volatile uint32_t never_set;          // the drain waits' stand-in for an abort flag
    __shared__ uint32_t issued_loads;               // k-block iterations whose loads the producer issued

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t stages = p.stages;
    if (p.k_splits > 1) launch_dependents();      // lets the reduce pass be scheduled while this grid runs

    if (threadIdx.x == 0) {
        abort_flag = 0;
        never_set = 0;
        issued_loads = 0;
        mbar_init(smem_u32(&drain_bar), 1);
        for (uint32_t s = 0; s < stages; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (uint32_t i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&tmem_full_bar[i]), 1);
            mbar_init(smem_u32(&tmem_empty_bar[i]), 8);   // one arrive per epilogue warp
        }
        fence_mbar_init();
        prefetch_tensormap(&tmap_a);
        prefetch_tensormap(&tmap_b);
        if (p.out_tma) prefetch_tensormap(&tmap_out);
    }
    if (warp == 1) {
        tmem_alloc_cta1(smem_u32(&tmem_holder), kTmemCols);
        tmem_relinquish_cta1();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_holder;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (elect_one()) {
            uint32_t stage = 0, phase = 0, issued = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
                const TileCoord tc = decode_tile(p, tile, BN);
                uint32_t batch = tc.batch, m0 = tc.m0, n0 = tc.n0;
                for (uint32_t kb = tc.kb0; kb < tc.kb1; ++kb) {
                    if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, &abort_flag, p.wait_cycles)) { ok = false; break; }
                    const uint32_t bar = smem_u32(&full_bar[stage]);
                    const uint32_t sa = smem_base + stage * kStageBytes;
                    const uint32_t sb = sa + kATileBytes;
                    const int32_t k0 = static_cast<int32_t>(kb * p.kb_elems);
                    mbar_arrive_expect_tx(bar, p.stage_tx_bytes);
                    if (!p.a.mn_major) {
                        tma_load_3d(sa, &tmap_a, bar, k0, m0, batch * p.a.batch_mul);
                    } else {
                        for (uint32_t c = 0; c < p.a.chunks; ++c)
                            tma_load_3d(sa + c * p.a.chunk_bytes, &tmap_a, bar, m0 + c * p.a.chunk_elems, k0,
                                        batch * p.a.batch_mul);
                    }
                    if (!p.b.mn_major) {
                        tma_load_3d(sb, &tmap_b, bar, k0, n0, batch * p.b.batch_mul);
                    } else {
                        for (uint32_t c = 0; c < p.b.chunks; ++c)
                            tma_load_3d(sb + c * p.b.chunk_bytes, &tmap_b, bar, n0 + c * p.b.chunk_elems, k0,
                                        batch * p.b.batch_mul);
                    }
                    ++issued;
                    if (++stage == stages) { stage = 0; phase ^= 1; }
                }
            }
            issued_loads = issued;
            if (!ok) {
                abort_flag = 1;
                atomicOr(&g_gemm_status, kStatusProducerTimeout);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            uint32_t stage = 0, phase = 0, local = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++local) {
                const uint32_t buf = local & 1;
                const uint32_t acc_phase = (local >> 1) & 1;
                if (!mbar_wait(smem_u32(&tmem_empty_bar[buf]), acc_phase ^ 1, &abort_flag, p.wait_cycles)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * BN;
                const TileCoord tc = decode_tile(p, tile, BN);
                for (uint32_t kb = tc.kb0; kb < tc.kb1; ++kb) {
                    if (!mbar_wait(smem_u32(&full_bar[stage]), phase, &abort_flag, p.wait_cycles)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t sa = smem_base + stage * kStageBytes;
                    const uint32_t sb = sa + kATileBytes;
                    const uint32_t a_lo = ((sa >> 4) & 0x3fffu) | p.a.desc_lo_fixed;
                    const uint32_t b_lo = ((sb >> 4) & 0x3fffu) | p.b.desc_lo_fixed;
#pragma unroll
                    for (uint32_t k = 0; k < kKStepsPerStage; ++k) {
                        const uint64_t adesc = (static_cast<uint64_t>(p.a.desc_hi) << 32) | (a_lo + k * p.a.kstep);
                        const uint64_t bdesc = (static_cast<uint64_t>(p.b.desc_hi) << 32) | (b_lo + k * p.b.kstep);
                        if constexpr (sizeof(T) == 4) umma_tf32_cta1(d_tmem, adesc, bdesc, p.idesc, (kb != tc.kb0 || k != 0));
                        else                          umma_f16_cta1(d_tmem, adesc, bdesc, p.idesc, (kb != tc.kb0 || k != 0));
                    }
                    umma_commit_cta1(smem_u32(&empty_bar[stage]));
                    if (++stage == stages) { stage = 0; phase ^= 1; }
                }
                if (ok) umma_commit_cta1(smem_u32(&tmem_full_bar[buf]));
            }
            if (!ok) {
                abort_flag = 1;
                atomicOr(&g_gemm_status, kStatusMmaTimeout);
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue
        const uint32_t quarter = warp & 3;       // TMEM lanes this warp may read
        uint32_t local = 0;
        bool ok = true;
        // The first pass of the loop is the rehearsal (see drain_accumulator): same call site, hence the same
        // instructions, on the second accumulator buffer, which nothing writes before the second tile.
        uint32_t rehearsal = (!GATHER && p.epilogue == kEpilogueStore) ? 1u : 0u;
        for (uint32_t tile = blockIdx.x; ok && tile < p.num_tiles;) {
            const TileCoord tc = decode_tile(p, tile, BN);
            uint32_t batch = tc.obatch, m0 = tc.m0, n0 = tc.n0;
            const uint32_t buf = rehearsal ? 1u : (local & 1);
            const uint32_t acc_phase = (local >> 1) & 1;
            TileBias<OutT, BN, 2> tile_bias = {};
            if (!rehearsal) {
                load_tile_bias<OutT, BN, 2>(p, (warp - 2) >> 2, quarter, lane, m0, n0, tile_bias);  // under the reduction
                if (!mbar_wait(smem_u32(&tmem_full_bar[buf]), acc_phase, &abort_flag, p.wait_cycles)) { ok = false; break; }
                tc_fence_after_sync();
            }
            if constexpr (GATHER)
                drain_accumulator<OutT, BN, false, 2, true>(p, &tmap_out, smem_base + stages * kStageBytes + (warp - 2) * 4096,
                                                            (warp - 2) >> 2, tmem_base + buf * BN, quarter, lane, batch, m0, n0,
                                                            tile_bias, 0, &peer_maps);
            else if (sizeof(OutT) == 2 && p.epilogue == kEpilogueLstm) {
                if constexpr (sizeof(OutT) == 2)
                    drain_accumulator_lstm<OutT, BN, 2>(p, (warp - 2) >> 2, tmem_base + buf * BN, quarter, lane, m0, n0);
            } else
                drain_accumulator<OutT, BN, false, 2>(p, &tmap_out, smem_base + stages * kStageBytes + (warp - 2) * 4096,
                                                      (warp - 2) >> 2, tmem_base + buf * BN, quarter, lane, batch, m0, n0, tile_bias,
                                                      0, nullptr, rehearsal);
            if (rehearsal) { rehearsal = 0; continue; }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[buf]));
            tile += gridDim.x;
            ++local;
        }
        drain_finish(lane);
        if (!ok) {
            abort_flag = 1;
            if (lane == 0) atomicOr(&g_gemm_status, kStatusEpilogueTimeout);
        }
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (abort_flag != 0) {
        if (warp == 0 && lane == 0) drain_armed_stages(full_bar, stages, issued_loads, &never_set);
        if (warp == 1 && lane == 0) {
            umma_commit_cta1(smem_u32(&drain_bar));
            mbar_wait(smem_u32(&drain_bar), 0, &never_set, kDrainCycles);
        }
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_cta1(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------------------------
// CTA-pair variant (tcgen05 cta_group::2): a cluster of two CTAs computes one 256 x BN tile.
// CTA r of the pair loads rows [m0 + 128 r, +128) of A and rows/columns [n0 + BN/2 r, +BN/2) of
// B, so every byte of the tile's operands is fetched once per pair (2/3 of the shared-memory
// fill traffic of two independent 128 x BN tiles).  One thread of CTA 0 issues the MMAs for
// both CTAs; each CTA's TMEM receives its own 128 rows of the accumulator and its own epilogue
// warps drain them.
//
// Synchronisation (stage s, accumulator buffer b):
//   full[s]      CTA 0 only: its producer arms it with the bytes of BOTH CTAs' loads; the loads
//                of CTA 1 complete their byte count on CTA 0's barrier (cta_group::2 form).
//   empty[s]     both CTAs, signalled together by one multicast tcgen05.commit of CTA 0.
//   tmem_full[b] both CTAs, multicast tcgen05.commit after the tile's last MMA.
//   tmem_empty[b] CTA 0 only, count 16: the eight epilogue warps of each CTA.
// No TMA load is multicast; all loads are plain per-CTA tile loads.
//
// GATHER: the epilogue also stores every tile into the peers' output buffers (product followed
// by an all-gather of the shards, in one kernel; see drain_accumulator).
template <typename T, uint32_t BN, bool GATHER = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmap_a,
                         const __grid_constant__ CUtensorMap tmap_b,
                         const __grid_constant__ CUtensorMap tmap_out,
                         const __grid_constant__ GemmParams p,
                         const __grid_constant__ typename PeerArgOf<GATHER>::type peer_maps)
{
    constexpr uint32_t kBHalf = BN / 2;
    constexpr uint32_t kBTileBytes = kBHalf * kRowBytes;
    constexpr uint32_t kStageBytes = kATileBytes + kBTileBytes;
    constexpr uint32_t kTmemCols = 2 * BN;
    constexpr uint32_t kMaxStages = 8;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

    __shared__ __align__(8) uint64_t full_bar[kMaxStages];
    __shared__ __align__(8) uint64_t empty_bar[kMaxStages];
    __shared__ __align__(8) uint64_t tmem_full_bar[2];
    __shared__ __align__(8) uint64_t tmem_empty_bar[2];
    __shared__ __align__(8) uint64_t drain_bar;
    __shared__ uint32_t tmem_holder;
    __shared__ volatile uint32_t abort_flag;
    __shared__ volatile uint32_t never_set;          // the drain waits' stand-in for an abort flag
    __shared__ uint32_t issued_loads;               // k-block iterations whose loads this CTA's producer issued

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t stages = p.stages;
    const uint32_t cta_rank = cluster_ctarank();          // 0 = leader
    const uint32_t pair_id = blockIdx.x >> 1;
    const uint32_t num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        never_set = 0;
        issued_loads = 0;
        mbar_init(smem_u32(&drain_bar), 1);
        for (uint32_t s = 0; s < stages; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (uint32_t i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&tmem_full_bar[i]), 1);
            mbar_init(smem_u32(&tmem_empty_bar[i]), 16);
        }
        fence_mbar_init();
        prefetch_tensormap(&tmap_a);
        prefetch_tensormap(&tmap_b);
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
    // a wait that gives up ends BOTH CTAs of the pair: the partner's waits see the flag at their next look
    auto raise_abort = [&](uint32_t code) {
        abort_flag = 1;
        st_shared_remote_u32(smem_u32(const_cast<uint32_t*>(&abort_flag)), cta_rank ^ 1u, 1u);
        atomicOr(&g_gemm_status, code);
    };
    // the loads of this CTA for k-block iteration j of the pair's work list (every tile has p.k_blocks of them:
    // pair tiles are never split along K); CTA 0 arms the stage's barrier for both CTAs
    auto issue_loads = [&](uint32_t j) {
        const uint32_t t_local = j / p.k_blocks, kb = j - t_local * p.k_blocks, stage = j % stages;
        const TileCoord tc = decode_tile(p, pair_id + t_local * num_pairs, BN);
        const uint32_t m0 = tc.m0 * 2 + cta_rank * kTileM, n0 = tc.n0 + cta_rank * kBHalf, batch = tc.batch;
        const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
        const uint32_t sa = smem_base + stage * kStageBytes;
        const uint32_t sb = sa + kATileBytes;
        const int32_t k0 = static_cast<int32_t>(kb * p.kb_elems);
        if (cta_rank == 0) mbar_arrive_expect_tx(smem_u32(&full_bar[stage]), 2 * p.stage_tx_bytes);
        if (!p.a.mn_major) {
            tma_load_3d_pair(sa, &tmap_a, bar, k0, m0, batch * p.a.batch_mul);
        } else {
            for (uint32_t c = 0; c < p.a.chunks; ++c)
                tma_load_3d_pair(sa + c * p.a.chunk_bytes, &tmap_a, bar, m0 + c * p.a.chunk_elems, k0, batch * p.a.batch_mul);
        }
        if (!p.b.mn_major) {
            tma_load_3d_pair(sb, &tmap_b, bar, k0, n0, batch * p.b.batch_mul);
        } else {
            for (uint32_t c = 0; c < p.b.chunks; ++c)
                tma_load_3d_pair(sb + c * p.b.chunk_bytes, &tmap_b, bar, n0 + c * p.b.chunk_elems, k0, batch * p.b.batch_mul);
        }
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        if (elect_one()) {
            uint32_t stage = 0, phase = 0, issued = 0;
            bool ok = true;
            for (uint32_t tile = pair_id; ok && tile < p.num_tiles; tile += num_pairs) {
                const TileCoord tc = decode_tile(p, tile, BN);
                uint32_t batch = tc.batch, m0 = tc.m0, n0 = tc.n0;
                m0 = m0 * 2 + cta_rank * kTileM;            // decode_tile counts 128-row units; pair tiles are 256 rows
                n0 += cta_rank * kBHalf;
                for (uint32_t kb = tc.kb0; kb < tc.kb1; ++kb) {
                    if (!mbar_wait_cluster(smem_u32(&empty_bar[stage]), phase ^ 1, &abort_flag, p.wait_cycles)) { ok = false; break; }
                    // every load of the pair reports to the leader's barrier
                    const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
                    const uint32_t sa = smem_base + stage * kStageBytes;
                    const uint32_t sb = sa + kATileBytes;
                    const int32_t k0 = static_cast<int32_t>(kb * p.kb_elems);
                    if (cta_rank == 0) mbar_arrive_expect_tx(smem_u32(&full_bar[stage]), 2 * p.stage_tx_bytes);
                    if (!p.a.mn_major) {
                        tma_load_3d_pair(sa, &tmap_a, bar, k0, m0, batch * p.a.batch_mul);
                    } else {
                        for (uint32_t c = 0; c < p.a.chunks; ++c)
                            tma_load_3d_pair(sa + c * p.a.chunk_bytes, &tmap_a, bar, m0 + c * p.a.chunk_elems, k0,
                                             batch * p.a.batch_mul);
                    }
                    if (!p.b.mn_major) {
                        tma_load_3d_pair(sb, &tmap_b, bar, k0, n0, batch * p.b.batch_mul);
                    } else {
                        for (uint32_t c = 0; c < p.b.chunks; ++c)
                            tma_load_3d_pair(sb + c * p.b.chunk_bytes, &tmap_b, bar, n0 + c * p.b.chunk_elems, k0,
                                             batch * p.b.batch_mul);
                    }
                    ++issued;
                    if (++stage == stages) { stage = 0; phase ^= 1; }
                }
            }
            issued_loads = issued;
            if (!ok) raise_abort(kStatusProducerTimeout);
        }
    } else if (warp == 1) {
        if (elect_one()) {
            uint32_t stage = 0, phase = 0, local = 0;
            bool ok = true;
            if (cta_rank == 0) {
                // -------------------------------------------------------------- MMA issuer (leader)
                for (uint32_t tile = pair_id; ok && tile < p.num_tiles; tile += num_pairs, ++local) {
                    const uint32_t buf = local & 1;
                    const uint32_t acc_phase = (local >> 1) & 1;
                    if (!mbar_wait_cluster(smem_u32(&tmem_empty_bar[buf]), acc_phase ^ 1, &abort_flag, p.wait_cycles)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + buf * BN;
                    const TileCoord tc = decode_tile(p, tile, BN);
                    for (uint32_t kb = tc.kb0; kb < tc.kb1; ++kb) {
                        if (!mbar_wait_cluster(smem_u32(&full_bar[stage]), phase, &abort_flag, p.wait_cycles)) { ok = false; break; }
                        tc_fence_after_sync();
                        const uint32_t sa = smem_base + stage * kStageBytes;
                        const uint32_t sb = sa + kATileBytes;
                        const uint32_t a_lo = ((sa >> 4) & 0x3fffu) | p.a.desc_lo_fixed;
                        const uint32_t b_lo = ((sb >> 4) & 0x3fffu) | p.b.desc_lo_fixed;
#pragma unroll
                        for (uint32_t k = 0; k < kKStepsPerStage; ++k) {
                            const uint64_t adesc = (static_cast<uint64_t>(p.a.desc_hi) << 32) | (a_lo + k * p.a.kstep);
                            const uint64_t bdesc = (static_cast<uint64_t>(p.b.desc_hi) << 32) | (b_lo + k * p.b.kstep);
                            if constexpr (sizeof(T) == 4) umma_tf32_cta2(d_tmem, adesc, bdesc, p.idesc, (kb != tc.kb0 || k != 0));
                            else                          umma_f16_cta2(d_tmem, adesc, bdesc, p.idesc, (kb != tc.kb0 || k != 0));
                        }
                        umma_commit_cta2_mc(smem_u32(&empty_bar[stage]), 3);
                        if (++stage == stages) { stage = 0; phase ^= 1; }
                    }
                    if (ok) umma_commit_cta2_mc(smem_u32(&tmem_full_bar[buf]), 3);
                }
                if (!ok) raise_abort(kStatusMmaTimeout);
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (both CTAs)
        const uint32_t quarter = warp & 3;
        uint32_t local = 0;
        bool ok = true;
        // first pass = rehearsal, as in gemm_tcgen05_kernel
        uint32_t rehearsal = (!GATHER && p.epilogue == kEpilogueStore) ? 1u : 0u;
        for (uint32_t tile = pair_id; ok && tile < p.num_tiles;) {
            const TileCoord tc = decode_tile(p, tile, BN);
            uint32_t batch = tc.obatch, m0 = tc.m0, n0 = tc.n0;
            m0 = m0 * 2 + cta_rank * kTileM;
            const uint32_t buf = rehearsal ? 1u : (local & 1);
            const uint32_t acc_phase = (local >> 1) & 1;
            TileBias<T, BN, 2> tile_bias = {};
            if (!rehearsal) {
                load_tile_bias<T, BN, 2>(p, (warp - 2) >> 2, quarter, lane, m0, n0, tile_bias);      // under the reduction
                if (!mbar_wait_cluster(smem_u32(&tmem_full_bar[buf]), acc_phase, &abort_flag, p.wait_cycles)) { ok = false; break; }
                tc_fence_after_sync();
            }
            if constexpr (GATHER)
                drain_accumulator<T, BN, false, 2, true>(p, &tmap_out, smem_base + stages * kStageBytes + (warp - 2) * 4096,
                                                         (warp - 2) >> 2, tmem_base + buf * BN, quarter, lane, batch, m0, n0,
                                                         tile_bias, 0, &peer_maps);
            else if (sizeof(T) == 2 && p.epilogue == kEpilogueLstm) {
                if constexpr (sizeof(T) == 2)
                    drain_accumulator_lstm<T, BN, 2>(p, (warp - 2) >> 2, tmem_base + buf * BN, quarter, lane, m0, n0);
            } else
                drain_accumulator<T, BN, false, 2>(p, &tmap_out, smem_base + stages * kStageBytes + (warp - 2) * 4096,
                                                   (warp - 2) >> 2, tmem_base + buf * BN, quarter, lane, batch, m0, n0, tile_bias,
                                                   0, nullptr, rehearsal);
            if (rehearsal) { rehearsal = 0; continue; }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(smem_u32(&tmem_empty_bar[buf]), 0);
            tile += num_pairs;
            ++local;
        }
        drain_finish(lane);
        if (!ok && lane == 0) raise_abort(kStatusEpilogueTimeout);
    }

    // ---------------------------------------------------------------------- teardown
    // no CTA may leave while its peer can still signal its barriers or read its shared memory
    tc_fence_before_sync();
    __syncwarp();
    cluster_arrive_release();
    cluster_wait_acquire();
    if (abort_flag != 0) {
        // Both CTAs take this branch (the flag is raised in both before the barrier above).  In order: the
        // leader waits for every MMA issued so far; the producer that issued fewer k-block iterations than its
        // partner issues the missing loads, so that every armed stage receives the bytes of both CTAs; the
        // leader waits for all armed stages.  After that nothing asynchronous targets either CTA.
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
        if (cta_rank == 0 && warp == 0 && lane == 0) drain_armed_stages(full_bar, stages, both, &never_set);
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

// ---------------------------------------------------------------------------------------------
// Float32 on the tensor cores: 3 x TF32.  A TF32 MMA reads fp32 words and uses the sign, the
// exponent and the top 10 mantissa bits.  Each operand x is split as x = hi + lo with
// hi = x with the low 13 mantissa bits cleared (exactly a TF32 value) and lo = x - hi (exact
// in fp32, at most 13 significant bits), and the product is accumulated as
//     hi_a.hi_b + hi_a.lo_b + lo_a.hi_b          (lo_a.lo_b ~ 2^-22 |a.b| is dropped)
// in two fp32 TMEM accumulators (dominant products / correction terms) that the epilogue sums.
// TMA delivers the raw fp32 tile, which serves as hi unchanged: the MMA ignores the low 13
// mantissa bits (truncation, confirmed by the 1e-5 parity tests -- rounding would show as 5e-4).
// Four transform warps write lo to a second buffer with the same (swizzled) layout, so the same
// shared-memory descriptors address both.
//   warp 0 producer, warp 1 MMA issuer, warps 2-5 epilogue, warps 6-13 transform.
//   full[s]  TMA bytes landed -> transform warps;  ready[s] (count 8) transform done -> MMA;
//   empty[s] MMAs done -> producer.
constexpr uint32_t kSplitTransformWarps = 8;   // two per scheduler: one warp alone issues too slowly
constexpr uint32_t kSplitThreads = (6 + kSplitTransformWarps) * 32;

template <uint32_t BN>
__global__ void __launch_bounds__(kSplitThreads, 1)
gemm_tcgen05_split_kernel(const __grid_constant__ CUtensorMap tmap_a,
                          const __grid_constant__ CUtensorMap tmap_b,
                          const __grid_constant__ CUtensorMap tmap_out,
                          const __grid_constant__ GemmParams p)
{
    using T = float;
    constexpr uint32_t kBTileBytes = BN * kRowBytes;
    constexpr uint32_t kHalfBytes = kATileBytes + kBTileBytes;     // hi tiles; lo tiles follow
    constexpr uint32_t kStageBytes = 2 * kHalfBytes;
    // two accumulators per tile (dominant products / correction terms); tiles are double-buffered
    // while 4 x BN columns fit in TMEM
    constexpr uint32_t kAccBufs = BN == 256 ? 1 : 2;
    constexpr uint32_t kTmemCols = kAccBufs * 2 * BN;
    constexpr uint32_t kMaxStages = 4;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

    __shared__ __align__(8) uint64_t full_bar[kMaxStages];
    __shared__ __align__(8) uint64_t ready_bar[kMaxStages];
    __shared__ __align__(8) uint64_t empty_bar[kMaxStages];
    __shared__ __align__(8) uint64_t tmem_full_bar[2];
    __shared__ __align__(8) uint64_t tmem_empty_bar[2];
    __shared__ __align__(8) uint64_t drain_bar;
    __shared__ uint32_t tmem_holder;
    __shared__ volatile uint32_t abort_flag;
    __shared__ volatile uint32_t never_set;          // the drain waits' stand-in for an abort flag
    __shared__ uint32_t issued_loads;               // k-block iterations whose loads the producer issued

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t stages = p.stages;
    if (p.k_splits > 1) launch_dependents();      // lets the reduce pass be scheduled while this grid runs

    if (threadIdx.x == 0) {
        abort_flag = 0;
        never_set = 0;
        issued_loads = 0;
        mbar_init(smem_u32(&drain_bar), 1);
        for (uint32_t s = 0; s < stages; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&ready_bar[s]), kSplitTransformWarps);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (uint32_t i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&tmem_full_bar[i]), 1);
            mbar_init(smem_u32(&tmem_empty_bar[i]), 4);
        }
        fence_mbar_init();
        prefetch_tensormap(&tmap_a);
        prefetch_tensormap(&tmap_b);
        if (p.out_tma) prefetch_tensormap(&tmap_out);
    }
    if (warp == 1) {
        tmem_alloc_cta1(smem_u32(&tmem_holder), kTmemCols);
        tmem_relinquish_cta1();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_holder;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (elect_one()) {
            uint32_t stage = 0, phase = 0, issued = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
                const TileCoord tc = decode_tile(p, tile, BN);
                uint32_t batch = tc.batch, m0 = tc.m0, n0 = tc.n0;
                for (uint32_t kb = tc.kb0; kb < tc.kb1; ++kb) {
                    if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, &abort_flag, p.wait_cycles)) { ok = false; break; }
                    const uint32_t bar = smem_u32(&full_bar[stage]);
                    const uint32_t sa = smem_base + stage * kStageBytes;
                    const uint32_t sb = sa + kATileBytes;
                    const int32_t k0 = static_cast<int32_t>(kb * p.kb_elems);
                    mbar_arrive_expect_tx(bar, p.stage_tx_bytes);
                    if (!p.a.mn_major) {
                        tma_load_3d(sa, &tmap_a, bar, k0, m0, batch * p.a.batch_mul);
                    } else {
                        for (uint32_t c = 0; c < p.a.chunks; ++c)
                            tma_load_3d(sa + c * p.a.chunk_bytes, &tmap_a, bar, m0 + c * p.a.chunk_elems, k0,
                                        batch * p.a.batch_mul);
                    }
                    if (!p.b.mn_major) {
                        tma_load_3d(sb, &tmap_b, bar, k0, n0, batch * p.b.batch_mul);
                    } else {
                        for (uint32_t c = 0; c < p.b.chunks; ++c)
                            tma_load_3d(sb + c * p.b.chunk_bytes, &tmap_b, bar, n0 + c * p.b.chunk_elems, k0,
                                        batch * p.b.batch_mul);
                    }
                    ++issued;
                    if (++stage == stages) { stage = 0; phase ^= 1; }
                }
            }
            issued_loads = issued;
            if (!ok) {
                abort_flag = 1;
                atomicOr(&g_gemm_status, kStatusProducerTimeout);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            uint32_t stage = 0, phase = 0, local = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++local) {
                const uint32_t buf = local % kAccBufs;
                const uint32_t acc_phase = (local / kAccBufs) & 1;
                if (!mbar_wait(smem_u32(&tmem_empty_bar[buf]), acc_phase ^ 1, &abort_flag, p.wait_cycles)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t d_main = tmem_base + buf * 2 * BN;
                const uint32_t d_small = d_main + BN;
                const TileCoord tc = decode_tile(p, tile, BN);
                for (uint32_t kb = tc.kb0; kb < tc.kb1; ++kb) {
                    if (!mbar_wait(smem_u32(&ready_bar[stage]), phase, &abort_flag, p.wait_cycles)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t sa = smem_base + stage * kStageBytes;
                    const uint32_t sb = sa + kATileBytes;
                    const uint32_t a_hi = ((sa >> 4) & 0x3fffu) | p.a.desc_lo_fixed;
                    const uint32_t b_hi = ((sb >> 4) & 0x3fffu) | p.b.desc_lo_fixed;
                    const uint32_t a_lo = (((sa + kHalfBytes) >> 4) & 0x3fffu) | p.a.desc_lo_fixed;
                    const uint32_t b_lo = (((sb + kHalfBytes) >> 4) & 0x3fffu) | p.b.desc_lo_fixed;
                    const uint64_t ahi64 = static_cast<uint64_t>(p.a.desc_hi) << 32;
                    const uint64_t bhi64 = static_cast<uint64_t>(p.b.desc_hi) << 32;
#pragma unroll
                    for (uint32_t k = 0; k < kKStepsPerStage; ++k) {
                        const uint32_t da = k * p.a.kstep, db = k * p.b.kstep;
                        // The accumulator add truncates toward zero, a bias that grows with the number
                        // of adds and with the accumulator's magnitude: the correction terms get their
                        // own (2^-11 times smaller) accumulator and are added once, in the epilogue.
                        umma_tf32_cta1(d_main, ahi64 | (a_hi + da), bhi64 | (b_hi + db), p.idesc, (kb != tc.kb0 || k != 0));
                        umma_tf32_cta1(d_small, ahi64 | (a_lo + da), bhi64 | (b_hi + db), p.idesc, (kb != tc.kb0 || k != 0));
                        umma_tf32_cta1(d_small, ahi64 | (a_hi + da), bhi64 | (b_lo + db), p.idesc, 1);
                    }
                    umma_commit_cta1(smem_u32(&empty_bar[stage]));
                    if (++stage == stages) { stage = 0; phase ^= 1; }
                }
                if (ok) umma_commit_cta1(smem_u32(&tmem_full_bar[buf]));
            }
            if (!ok) {
                abort_flag = 1;
                atomicOr(&g_gemm_status, kStatusMmaTimeout);
            }
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------------ epilogue
        const uint32_t quarter = warp & 3;
        uint32_t local = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++local) {
            const TileCoord tc = decode_tile(p, tile, BN);
            uint32_t batch = tc.obatch, m0 = tc.m0, n0 = tc.n0;
            const uint32_t buf = local % kAccBufs;
            const uint32_t acc_phase = (local / kAccBufs) & 1;
            TileBias<T, BN, 1> tile_bias;
            load_tile_bias<T, BN, 1>(p, 0, quarter, lane, m0, n0, tile_bias);                        // under the reduction
            if (!mbar_wait(smem_u32(&tmem_full_bar[buf]), acc_phase, &abort_flag, p.wait_cycles)) { ok = false; break; }
            tc_fence_after_sync();
            drain_accumulator<T, BN, true, 1>(p, &tmap_out, smem_base + stages * kStageBytes + (warp - 2) * 4096, 0,
                                              tmem_base + buf * 2 * BN, quarter, lane, batch, m0, n0, tile_bias,
                                              tmem_base + buf * 2 * BN + BN);
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[buf]));
        }
        drain_finish(lane);
        if (!ok) {
            abort_flag = 1;
            if (lane == 0) atomicOr(&g_gemm_status, kStatusEpilogueTimeout);
        }
    } else {
        // ------------------------------------------------------------------ hi / lo transform
        const uint32_t t = threadIdx.x - 6 * 32;              // 0 .. 32 * kSplitTransformWarps - 1
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
            const TileCoord tc = decode_tile(p, tile, BN);
            for (uint32_t kb = tc.kb0; kb < tc.kb1; ++kb) {
                if (!mbar_wait(smem_u32(&full_bar[stage]), phase, &abort_flag, p.wait_cycles)) { ok = false; break; }
                const uint32_t hi_base = smem_base + stage * kStageBytes;
#pragma unroll 4
                for (uint32_t off = t * 16; off < kHalfBytes; off += kSplitTransformWarps * 32 * 16) {
                    uint32_t x0, x1, x2, x3;
                    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(x0), "=r"(x1), "=r"(x2), "=r"(x3) : "r"(hi_base + off));
                    uint32_t x[4] = {x0, x1, x2, x3};
                    uint32_t l[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) l[j] = __float_as_uint(tf32_low_part(x[j]));
                    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};"
                                 ::"r"(hi_base + kHalfBytes + off), "r"(l[0]), "r"(l[1]), "r"(l[2]), "r"(l[3]) : "memory");
                }
                fence_proxy_async_smem();          // make the generic-proxy writes visible to the MMA
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&ready_bar[stage]));
                if (++stage == stages) { stage = 0; phase ^= 1; }
            }
        }
        if (!ok) {
            abort_flag = 1;
            if (lane == 0) atomicOr(&g_gemm_status, kStatusPairTimeout);
        }
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (abort_flag != 0) {
        if (warp == 0 && lane == 0) drain_armed_stages(full_bar, stages, issued_loads, &never_set);
        if (warp == 1 && lane == 0) {
            umma_commit_cta1(smem_u32(&drain_bar));
            mbar_wait(smem_u32(&drain_bar), 0, &never_set, kDrainCycles);
        }
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_cta1(tmem_base, kTmemCols);
    }
}

}  // namespace srt
