// C ABI of the B200 matmul path: argument validation, plan selection, TMA descriptor
// construction and kernel launches.  Declarations and the reference interfaces they replace
// are in include/srt_matmul_api.h.
#include "srt_matmul_api.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <vector>

#include "dense_backward.cuh"
#include "gemm_simt.cuh"
#include "gemm_splitk.cuh"
#include "gemm_tcgen05.cuh"
#include "gemm_tf32x3.cuh"
#include "lstm_cell.cuh"
#include "matrix_transform.cuh"

namespace {

using namespace srt;

thread_local char g_error[512] = "";
std::atomic<uint64_t> g_launches{0};
std::atomic<uint64_t> g_wait_limit_ns{srt::kDefaultWaitLimitNs};     // srtMatmulSetWaitLimit

struct Tuning {
    std::atomic<int32_t> force_kernel{0}, tile_n{0}, stages{0}, max_ctas{0}, split_k{0};
} g_tuning;

cudaError_t fail(cudaError_t code, const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
    return code;
}

// ------------------------------------------------------------------ the device of a call
// Every entry point that takes a stream works on THAT stream's device, whatever device is current
// on the calling thread: the reference's queues never select a device before they enqueue
// (Sources/SwiftRTCore/platform/cuda/functions/CudaMath.swift:117-125 launches on `stream` with no
// device call; nothing calls CudaQueue.selectDevice, cuda/device/CudaQueue.swift:77).  The scope
// resolves the stream's device, makes it current for the duration of the call when it differs and
// restores the caller's device afterwards; per-device state (workspaces, kernel attributes, the
// status word, the static scratch) is keyed by `device`.  The legacy and per-thread default
// streams belong to whatever device is current.  While a stream is being captured the runtime
// refuses the device query (and a refused call would invalidate the capture), so a capturing
// stream is taken to belong to the current device: capture with the stream's device current.
struct DeviceScope {
    int device = -1;
    int previous = -1;
    cudaError_t status = cudaSuccess;
    explicit DeviceScope(cudaStream_t stream)
    {
        int cur = 0;
        status = cudaGetDevice(&cur);
        if (status != cudaSuccess) return;
        int dev = cur;
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (stream != nullptr && stream != cudaStreamLegacy && stream != cudaStreamPerThread &&
            cudaStreamIsCapturing(stream, &cap) == cudaSuccess && cap == cudaStreamCaptureStatusNone) {
            status = cudaStreamGetDevice(stream, &dev);
            if (status != cudaSuccess) {
                fail(status, "cannot resolve the device of the stream: %s", cudaGetErrorString(status));
                return;
            }
        }
        device = dev;
        if (dev != cur) {
            status = cudaSetDevice(dev);
            if (status == cudaSuccess) previous = cur;
        }
    }
    ~DeviceScope()
    {
        if (previous >= 0) cudaSetDevice(previous);
    }
    DeviceScope(const DeviceScope&) = delete;
    DeviceScope& operator=(const DeviceScope&) = delete;
};

// ------------------------------------------------------------------ problem description
struct Problem {
    srtDataType type;
    uint32_t elem;                 // bytes per element
    uint64_t batch, M, N, K;
    const char* a; const char* b; char* out;
    long long a_b, a_m, a_k;       // element strides of op(a): batch, row, reduction
    long long b_b, b_k, b_n;
    long long o_b, o_m, o_n;
    const char* bias; long long bias_stride;
    uint32_t act;
};

uint32_t elem_size(srtDataType t)
{
    switch (t) {
    case real32F: return 4;
    case real16F: case real16BF: return 2;
    default: return 0;
    }
}

cudaError_t parse(const void* a, const srtTensorDescriptor* ad, bool ta,
                  const void* b, const srtTensorDescriptor* bd, bool tb,
                  const void* bias, const srtTensorDescriptor* biasd, int act,
                  const void* out, const srtTensorDescriptor* od, Problem& P)
{
    if (!ad || !bd || !od) return fail(cudaErrorInvalidValue, "null tensor or descriptor");
    if (!ad->shape || !ad->strides || !bd->shape || !bd->strides || !od->shape || !od->strides)
        return fail(cudaErrorInvalidValue, "descriptor without shape or strides");
    // tensors without elements have no storage to point at
    if ((!a && ad->count != 0) || (!b && bd->count != 0) || (!out && od->count != 0))
        return fail(cudaErrorInvalidValue, "null tensor or descriptor");
    if (ad->type != od->type || bd->type != od->type)
        return fail(cudaErrorInvalidValue, "a, b and out must have the same element type");
    P.type = od->type;
    P.elem = elem_size(P.type);
    if (P.elem == 0) return fail(cudaErrorNotSupported, "element type %d is not computed by this library", (int)P.type);
    if ((int)ad->order > 1 || (int)bd->order > 1 || (int)od->order > 1)
        return fail(cudaErrorNotSupported, "tiled storage orders are not supported");
    if (od->rank != 2 && od->rank != 3) return fail(cudaErrorNotSupported, "out must have rank 2 or 3");
    if (ad->rank < 2 || ad->rank > od->rank || bd->rank < 2 || bd->rank > od->rank)
        return fail(cudaErrorInvalidValue, "input rank must be 2 or the rank of out");

    const uint32_t oq = od->rank - 2, aq = ad->rank - 2, bq = bd->rank - 2;
    P.batch = od->rank == 3 ? od->shape[0] : 1;
    P.M = od->shape[oq];
    P.N = od->shape[oq + 1];
    const uint64_t a_rows = ad->shape[aq], a_cols = ad->shape[aq + 1];
    const uint64_t b_rows = bd->shape[bq], b_cols = bd->shape[bq + 1];
    const uint64_t aM = ta ? a_cols : a_rows, aK = ta ? a_rows : a_cols;
    const uint64_t bK = tb ? b_cols : b_rows, bN = tb ? b_rows : b_cols;
    if (aK != bK) return fail(cudaErrorInvalidValue, "matmul inner dimensions must be equal (%llu vs %llu)",
                              (unsigned long long)aK, (unsigned long long)bK);
    if (aM != P.M || bN != P.N)
        return fail(cudaErrorInvalidValue, "out shape [%llu x %llu] does not match op(a).op(b) [%llu x %llu]",
                    (unsigned long long)P.M, (unsigned long long)P.N, (unsigned long long)aM, (unsigned long long)bN);
    P.K = aK;
    // empty results (M, N or batch = 0) are accepted and launch nothing (see is_empty); an empty
    // reduction (K = 0) is a sum of no terms: out = activation(0 + bias), computed by the strided kernel
    const uint64_t lim = 0x7fffffffull;       // the reference limits dims to Int32.max (MatrixLayout.swift:117-142)
    if (P.M > lim || P.N > lim || P.K > lim || P.batch > 65535)
        return fail(cudaErrorInvalidValue, "dimension exceeds the supported range");

    P.a_m = (long long)(ta ? ad->strides[aq + 1] : ad->strides[aq]);
    P.a_k = (long long)(ta ? ad->strides[aq] : ad->strides[aq + 1]);
    P.b_k = (long long)(tb ? bd->strides[bq + 1] : bd->strides[bq]);
    P.b_n = (long long)(tb ? bd->strides[bq] : bd->strides[bq + 1]);
    P.o_m = (long long)od->strides[oq];
    P.o_n = (long long)od->strides[oq + 1];
    P.a_b = P.b_b = P.o_b = 0;
    if (od->rank == 3) {
        P.o_b = (long long)od->strides[0];
        if (ad->rank == 3) {
            if (ad->shape[0] != P.batch && ad->shape[0] != 1) return fail(cudaErrorInvalidValue, "batch size of a does not match out");
            P.a_b = ad->shape[0] == 1 ? 0 : (long long)ad->strides[0];
        }
        if (bd->rank == 3) {
            if (bd->shape[0] != P.batch && bd->shape[0] != 1) return fail(cudaErrorInvalidValue, "batch size of b does not match out");
            P.b_b = bd->shape[0] == 1 ? 0 : (long long)bd->strides[0];
        }
    }
    if ((P.M > 1 && P.o_m == 0) || (P.N > 1 && P.o_n == 0) || (P.batch > 1 && P.o_b == 0))
        return fail(cudaErrorInvalidValue, "out must not repeat elements (zero stride)");
    P.a = static_cast<const char*>(a);
    P.b = static_cast<const char*>(b);
    P.out = static_cast<char*>(const_cast<void*>(out));

    P.bias = nullptr;
    P.bias_stride = 0;
    if (bias) {
        if (!biasd || !biasd->shape || !biasd->strides) return fail(cudaErrorInvalidValue, "bias without descriptor");
        if (biasd->type != P.type) return fail(cudaErrorInvalidValue, "bias must have the element type of out");
        if (biasd->rank != 1 || biasd->shape[0] != P.N)
            return fail(cudaErrorInvalidValue, "bias must be rank 1 with %llu elements", (unsigned long long)P.N);
        P.bias = static_cast<const char*>(bias);
        P.bias_stride = (long long)biasd->strides[0];
    }
    switch (act) {
    case srtActivationSigmoid: case srtActivationRelu: case srtActivationTanh:
    case srtActivationIdentity: case srtActivationGelu: case srtActivationGeluTanh:
        P.act = (uint32_t)act;
        break;
    case srtActivationClippedRelu: case srtActivationElu:
        return fail(cudaErrorNotSupported, "clippedRelu and elu need coefficients that this entry point does not carry");
    default:
        return fail(cudaErrorInvalidValue, "unknown activation %d", act);
    }
    g_error[0] = 0;
    return cudaSuccess;
}

// ------------------------------------------------------------------ per-device state
inline bool is_empty(const Problem& P) { return P.M == 0 || P.N == 0 || P.batch == 0; }

// ------------------------------------------------------------------ tuning choices and the plan table
// What the planner may be told instead of deciding by its cost model: 0 = decide.
struct Choice { int32_t force, tile_n, stages, max_ctas, split_k; };

// Set by srtMatmulTune while it times a candidate on this thread.
thread_local const Choice* t_choice_override = nullptr;

// Tuned choices by problem signature: sizes, element type and which strides are 1 (majorness of
// the operands and order of the output).  Filled by srtMatmulTune / srtMatmulPlanCacheLoad and
// consulted whenever no process-wide tuning is set.
struct PlanKey {
    int32_t type;
    uint32_t flags;                // bit 0 a_k == 1, 1 a_m == 1, 2 b_n == 1, 3 b_k == 1, 4 o_n == 1, 5 o_m == 1, 6 bias
    uint64_t M, N, K, batch;
};
struct PlanEntry { PlanKey key; Choice choice; float us; };
std::mutex g_plan_mutex;
std::vector<PlanEntry> g_plan_table;
std::atomic<uint32_t> g_plan_epoch{0};      // part of the call-cache key: bumps invalidate cached launches
std::once_flag g_plan_env_once;

PlanKey plan_key(const Problem& P)
{
    PlanKey k;
    memset(&k, 0, sizeof k);
    k.type = (int32_t)P.type;
    k.flags = (P.a_k == 1 ? 1u : 0u) | (P.a_m == 1 ? 2u : 0u) | (P.b_n == 1 ? 4u : 0u) | (P.b_k == 1 ? 8u : 0u) |
              (P.o_n == 1 ? 16u : 0u) | (P.o_m == 1 ? 32u : 0u) | (P.bias ? 64u : 0u);
    k.M = P.M; k.N = P.N; k.K = P.K; k.batch = P.batch;
    return k;
}

int plan_table_load(const char* path);      // defined with the entry points

bool plan_lookup(const Problem& P, Choice& out)
{
    std::call_once(g_plan_env_once, [] {
        const char* path = getenv("SRT_MATMUL_PLAN_CACHE");
        if (path && *path) plan_table_load(path);
    });
    const PlanKey k = plan_key(P);
    std::lock_guard<std::mutex> lock(g_plan_mutex);
    for (const PlanEntry& e : g_plan_table)
        if (memcmp(&e.key, &k, sizeof k) == 0) { out = e.choice; return true; }
    return false;
}

void plan_store(const PlanKey& k, const Choice& c, float us)
{
    std::lock_guard<std::mutex> lock(g_plan_mutex);
    for (PlanEntry& e : g_plan_table)
        if (memcmp(&e.key, &k, sizeof k) == 0) { e.choice = c; e.us = us; return; }
    g_plan_table.push_back(PlanEntry{k, c, us});
}

// The choice a plan is made under: the tuner's candidate, else the process-wide tuning, else a
// tuned entry of the plan table, else all zeros (the cost model decides).
Choice effective_choice(const Problem& P)
{
    if (t_choice_override) return *t_choice_override;
    Choice c = {g_tuning.force_kernel.load(), g_tuning.tile_n.load(), g_tuning.stages.load(), g_tuning.max_ctas.load(),
                g_tuning.split_k.load()};
    if (c.force == 0 && c.tile_n == 0 && c.stages == 0 && c.max_ctas == 0 && c.split_k == 0) {
        Choice tuned;
        if (plan_lookup(P, tuned)) return tuned;
    }
    return c;
}

struct DeviceInfo {
    int sms = 0;
    bool sm100 = false;
    bool attrs_set = false;
};
std::mutex g_mutex;
DeviceInfo g_devices[64];

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

cudaError_t device_info(int dev, DeviceInfo& out)
{
    std::lock_guard<std::mutex> lock(g_mutex);
    if (dev < 0 || dev >= 64) return fail(cudaErrorInvalidDevice, "device ordinal %d out of range", dev);
    DeviceInfo& d = g_devices[dev];
    if (d.sms == 0) {
        int major = 0, sms = 0;
        cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        if (e != cudaSuccess) return e;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return e;
        d.sm100 = (major == 10);
        d.sms = sms;
    }
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
            return fail(cudaErrorNotSupported, "driver does not export cuTensorMapEncodeTiled");
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    out = d;
    return cudaSuccess;
}

// ------------------------------------------------------------------ planning
struct TcOperand {
    bool ok = false;
    bool mn_major = false;
    long long ld = 0;          // elements between consecutive indices of the non-contiguous dim
};

// Can TMA address op(x) [rows x K] with element strides (s_r, s_k), batch stride s_b?
TcOperand classify(const char* ptr, uint64_t rows, uint64_t K, uint64_t batch, long long s_r, long long s_k,
                   long long s_b, uint32_t elem)
{
    TcOperand r;
    if (reinterpret_cast<uintptr_t>(ptr) % 16) return r;
    const bool k_unit = (s_k == 1 || K == 1), r_unit = (s_r == 1 || rows == 1);
    auto ok_stride = [&](long long s, uint64_t extent_inner) {
        return s > 0 && (s * (long long)elem) % 16 == 0 && (uint64_t)s >= extent_inner &&
               (unsigned long long)s * elem < (1ull << 40);
    };
    if (batch > 1 && s_b != 0 && !((s_b * (long long)elem) % 16 == 0 && s_b > 0 && (unsigned long long)s_b * elem < (1ull << 40)))
        return r;
    if (k_unit && (rows == 1 || ok_stride(s_r, K))) {
        r.ok = true; r.mn_major = false; r.ld = rows == 1 ? (long long)((K * elem + 15) / 16 * 16 / elem) : s_r;
        return r;
    }
    if (r_unit && (K == 1 || ok_stride(s_k, rows))) {
        r.ok = true; r.mn_major = true; r.ld = K == 1 ? (long long)((rows * elem + 15) / 16 * 16 / elem) : s_k;
        return r;
    }
    return r;
}

// 64 x 64 tiles unless such a grid would leave most SMs idle: then 32 x 32 (4x the blocks)
uint32_t simt_tile_for(uint64_t M, uint64_t N, uint64_t batch, int sms)
{
    const uint64_t t64 = ((M + 63) / 64) * ((N + 63) / 64) * batch;
    return t64 < (uint64_t)sms ? 32u : 64u;
}

struct Plan {
    srtMatmulPlan pub;
    bool swapped = false;
    Problem Q;                 // the problem as the kernel sees it (after a possible swap)
    TcOperand ta, tb;
    uint32_t bias_mode = 0;
    uint32_t splits = 1, kb_per_split = 0;   // split-K: partial sums in an fp32 workspace + a reduce pass
};

// `skinny_swap`: plan the transposed problem out^T = op(b)^T . op(a)^T although `out` is row-major, so
// that the wide dimension fills the 128 rows of the MMA and the few rows of `out` become its N.  Only
// valid when the plan ends up with split-K, whose reduce pass writes through any output strides;
// returns false (plan unusable) otherwise.
constexpr uint64_t kSkinnyRows = 256;     // up to this many rows the transposed plan is tried

bool make_plan_impl(const Problem& P, const DeviceInfo& dev, Plan& plan, bool skinny_swap)
{
    memset(&plan.pub, 0, sizeof plan.pub);
    plan.Q = P;
    plan.swapped = false;
    plan.bias_mode = P.bias ? 1 : 0;
    const Choice choice = effective_choice(P);
    const int32_t force = choice.force;

    bool tc = dev.sm100 && force != srtMatmulKernelSimt && P.K > 0;
    // the tensor-core path writes rows of contiguous columns; a col-order out is computed
    // as out^T = op(b)^T . op(a)^T, which is the same memory
    Problem Q = P;
    if (tc) {
        if (!skinny_swap && (P.o_n == 1 || P.N == 1)) {
            // as is
        } else if (skinny_swap || P.o_m == 1 || P.M == 1) {
            Q.M = P.N; Q.N = P.M;
            Q.a = P.b; Q.a_b = P.b_b; Q.a_m = P.b_n; Q.a_k = P.b_k;
            Q.b = P.a; Q.b_b = P.a_b; Q.b_k = P.a_k; Q.b_n = P.a_m;
            Q.o_m = P.o_n; Q.o_n = P.o_m;
            plan.swapped = true;
            if (P.bias) plan.bias_mode = 2;
        } else {
            tc = false;
        }
    }
    if (tc) {
        plan.ta = classify(Q.a, Q.M, Q.K, Q.batch, Q.a_m, Q.a_k, Q.a_b, Q.elem);
        plan.tb = classify(Q.b, Q.N, Q.K, Q.batch, Q.b_n, Q.b_k, Q.b_b, Q.elem);
        if (!plan.ta.ok || !plan.tb.ok) tc = false;
        if (!skinny_swap && Q.N > 1 && Q.o_m < (long long)Q.N && Q.M > 1) tc = false;   // overlapping output rows
    }
    // Float32 runs on the tensor cores as 3 x TF32 once the problem is large enough to pay for
    // it; below that the strided kernel is as fast and keeps the reference's exact arithmetic
    // The tensor cores add into the fp32 accumulator with truncation, an error that grows
    // linearly with K (measured 9e-7 at K = 256, 2.6e-6 at K = 1024, relative Frobenius):
    // beyond K = 2048 the reduction is cut into chunks of 2048 whose fp32 partial sums are added
    // in a second pass (split-K), which keeps the 1e-5 tolerance for any K.
    const bool split = tc && Q.type == real32F;
    if (split && force == 0 && Q.M * Q.N * Q.K * Q.batch < (1ull << 26)) tc = false;
    // tiny problems are launch-bound either way; keep them on the exact kernel
    if (tc && force == 0 && Q.M * Q.N * Q.K * Q.batch < (1ull << 18)) tc = false;

    // Float32 with a streamed, K-contiguous op(a) and a smaller op(b): the CTA-pair kernel that reads
    // op(a) once, multiplies TF32 + BFloat16 corrections and takes op(b) pre-split from a pack pass
    // (gemm_tf32x3.cuh).  K <= 2048 for the same accuracy reason as below; longer reductions go
    // through split-K on the one-CTA kernel.
    if (tc && split && !skinny_swap && (force == 0 || force == srtMatmulKernelTf32x3Pair) && !plan.ta.mn_major &&
        Q.K <= 2048 && Q.K >= 32 && Q.M >= Q.N && Q.N > 128 && Q.M >= 512 && choice.split_k <= 1 &&
        (force == srtMatmulKernelTf32x3Pair || Q.M * Q.N * Q.K * Q.batch >= (1ull << 28))) {
        const uint64_t kp = (Q.K + 31) / 32 * 32;
        const uint64_t b_items = (Q.batch == 1 || Q.b_b == 0) ? 1 : Q.batch;
        const uint64_t pack_bytes = b_items * ((Q.N + 127) / 128 * 128) * kp * 8;
        if (pack_bytes <= (256ull << 20)) {
            plan.Q = Q;
            // 256 x 256 tiles by default (three stages, exposed epilogue: 141 us on 65536 x 1024 x 256); 256 x 128 tiles
            // (four stages, the epilogue under the next tile's reduction: 161 us there) on request
            const uint32_t bn = choice.tile_n == 128 ? 128u : 256u;
            const uint64_t tiles = ((Q.M + 255) / 256) * ((Q.N + bn - 1) / bn) * Q.batch;
            const uint64_t pairs = (uint64_t)dev.sms / 2;
            uint32_t ctas = 2u * (uint32_t)(tiles < pairs ? tiles : pairs);
            if (choice.max_ctas > 1 && ctas > (uint32_t)choice.max_ctas) ctas = (uint32_t)choice.max_ctas & ~1u;
            plan.splits = 1;
            plan.kb_per_split = (uint32_t)(kp / 32);
            plan.pub.kernel = srtMatmulKernelTf32x3Pair;
            plan.pub.tileM = 256; plan.pub.tileN = (int32_t)bn; plan.pub.tileK = 32;
            plan.pub.stages = (int32_t)x3_stages(bn);
            plan.pub.ctas = (int32_t)ctas;
            plan.pub.tiles = (int32_t)tiles;
            plan.pub.swapped = plan.swapped;
            plan.pub.aMajor = 0; plan.pub.bMajor = 0;
            plan.pub.fp32Split = 1;
            plan.pub.splitK = 1;
            plan.pub.workspaceBytes = (size_t)pack_bytes;
            plan.pub.dynamicSmemBytes = (size_t)x3_smem_bytes(bn);
            return true;
        }
    }

    if (!tc) {
        plan.Q = P;
        plan.swapped = false;
        plan.bias_mode = P.bias ? 1 : 0;
        plan.pub.kernel = srtMatmulKernelSimt;
        const uint32_t st = simt_tile_for(P.M, P.N, P.batch, dev.sms);
        plan.pub.tileM = (int32_t)st; plan.pub.tileN = (int32_t)st; plan.pub.tileK = st == 32 ? 32 : kSimtK;
        plan.pub.stages = 1;
        const uint64_t tm = (P.M + st - 1) / st, tn = (P.N + st - 1) / st;
        plan.pub.tiles = (int32_t)(tm * tn * P.batch);
        plan.pub.ctas = plan.pub.tiles;
        plan.pub.dynamicSmemBytes = 0;
        return !skinny_swap;
    }

    plan.Q = Q;
    uint32_t bn = (uint32_t)choice.tile_n;
    // Tile choice by a small cost model: time ~ waves x (time of one tile).  A 128 x BN tile costs
    // BN / efficiency(BN) (narrow MMAs re-read A more often per flop); a CTA pair's 256 x BN tile
    // costs about the same as one CTA's 128 x BN tile and fills the device with half as many tiles.
    // (the 3 x TF32 kernel gets a third pipeline stage at BN = 128, which makes its narrow tile cheaper)
    auto tile_cost = [&](uint32_t n) {
        if (split) return n == 256 ? 256.0 : n == 128 ? 140.0 : 110.0;
        return n == 256 ? 256.0 : n == 128 ? 171.0 : 128.0;
    };
    auto waves = [](uint64_t tiles, uint64_t units) { return (double)((tiles + units - 1) / units); };
    auto tiles_for = [&](uint32_t tm, uint32_t n) { return ((Q.M + tm - 1) / tm) * ((Q.N + n - 1) / n) * Q.batch; };
    const uint64_t sms = (uint64_t)dev.sms;
    auto best_single = [&](uint32_t& n_out) {
        double best = 1e300;
        for (uint32_t n : {256u, 128u, 64u}) {
            if (n > 64 && Q.N <= n / 2) continue;                       // mostly padding
            const double c = waves(tiles_for(kTileM, n), sms) * tile_cost(n);
            if (c < best) { best = c; n_out = n; }
        }
        return best;
    };
    bool pair = false;
    if (split) {
        pair = false;
        if (bn != 64 && bn != 128 && bn != 256) best_single(bn);
    } else if (force == srtMatmulKernelTcgen05Pair) {
        pair = true;
        if (bn != 128 && bn != 256) bn = Q.N <= 128 ? 128 : 256;
    } else if (skinny_swap) {
        pair = false;
        bn = Q.N <= 64 ? 64 : Q.N <= 128 ? 128 : 256;                   // one column tile holds all the rows of the result
    } else if (bn == 64 || bn == 128 || bn == 256) {
        pair = false;                                                   // explicit single-CTA tile width
    } else {
        uint32_t n1 = 256;
        const double single = best_single(n1);
        bn = n1;
        // pairs pay off in long main loops; short ones are bound by the epilogue, where two
        // independent CTAs drain faster
        if (force == 0 && Q.M > kTileM && Q.K >= 1024 && Q.N > 128) {
            const double paired = waves(tiles_for(2 * kTileM, 256), sms / 2) * tile_cost(256) / 1.05;
            if (paired <= single) { pair = true; bn = 256; }
        }
    }
    const uint32_t tile_m = pair ? 2 * kTileM : kTileM;
    const bool split3 = split;
    const uint32_t stage_bytes = (kATileBytes + (pair ? bn / 2 : bn) * kRowBytes) * (split3 ? 2 : 1);
    uint32_t stages = (uint32_t)choice.stages;
    uint32_t max_stages = (227u * 1024u - 2048u - kEpilogueStagingBytes) / stage_bytes;
    if (split3 && max_stages > 4) max_stages = 4;
    // Four 32 KB stages keep the pair kernel's MMAs fed; deeper rings measured slower on a
    // power-capped B200 (higher pipe utilisation, lower clock, lower L2 hit rate).
    if (stages < 2 || stages > 8) {
        // a single wave of pair tiles starts cold on every SM at once and is bound by load latency: six stages
        // (36.9 us against 39.7 us on the Dense configuration); in a long run of waves four are faster (above)
        const uint64_t pair_tiles = ((Q.M + 2 * kTileM - 1) / (2 * kTileM)) * ((Q.N + bn - 1) / bn) * Q.batch;
        stages = pair ? (pair_tiles <= sms / 2 ? 6 : 4) : 8;
    }
    if (stages > max_stages) stages = max_stages;
    const uint32_t kb_elems = kRowBytes / Q.elem;
    const uint64_t tiles_m = (Q.M + tile_m - 1) / tile_m, tiles_n = (Q.N + bn - 1) / bn;
    const uint64_t tiles = tiles_m * tiles_n * Q.batch;
    // split-K: (1) Float32 beyond K = 2048, for accuracy; (2) few tiles and a long reduction, to
    // give every SM work.  Partial sums go to an fp32 workspace [split][batch][M][N].
    const uint32_t k_blocks = (uint32_t)((Q.K + kb_elems - 1) / kb_elems);
    uint32_t splits = 1, kb_per_split = k_blocks;
    const int32_t want_split = choice.split_k;
    if (!pair && want_split != 1) {
        uint32_t target = 1;
        if (want_split > 1) target = (uint32_t)want_split;
        else {
            if (split3 && Q.K > 2048) target = (uint32_t)((Q.K + 2047) / 2048);
            if (tiles * 2 <= sms && k_blocks >= 32) {
                uint32_t occ = (uint32_t)(sms / tiles);
                if (occ > k_blocks / 16) occ = k_blocks / 16;
                if (occ > 32) occ = 32;
                if (occ > target) target = occ;
            }
        }
        if (target > k_blocks) target = k_blocks;
        if (target > 1) {
            kb_per_split = (k_blocks + target - 1) / target;
            if (split3 && kb_per_split * kb_elems > 2048) kb_per_split = 2048 / kb_elems;
            splits = (k_blocks + kb_per_split - 1) / kb_per_split;
        }
        const uint64_t ws_bytes = (uint64_t)splits * Q.batch * Q.M * Q.N * 4;
        if (splits > 1 && ws_bytes > (2ull << 30)) {
            if (split3 && Q.K > 2048 && want_split == 0) {       // cannot hold the tolerance without it
                plan.Q = P; plan.swapped = false; plan.bias_mode = P.bias ? 1 : 0;
                plan.pub.kernel = srtMatmulKernelSimt;
                const uint32_t st = simt_tile_for(P.M, P.N, P.batch, dev.sms);
                plan.pub.tileM = (int32_t)st; plan.pub.tileN = (int32_t)st; plan.pub.tileK = st == 32 ? 32 : kSimtK;
                plan.pub.stages = 1;
                plan.pub.tiles = (int32_t)(((P.M + st - 1) / st) * ((P.N + st - 1) / st) * P.batch);
                plan.pub.ctas = plan.pub.tiles;
                return !skinny_swap;
            }
            splits = 1; kb_per_split = k_blocks;
        }
    }
    plan.splits = splits;
    plan.kb_per_split = kb_per_split;
    const uint64_t work_units = tiles * splits;
    const uint64_t units = pair ? (uint64_t)dev.sms / 2 : (uint64_t)dev.sms;   // CTAs or CTA pairs
    uint32_t ctas = (uint32_t)(work_units < units ? work_units : units);
    const int32_t cap = choice.max_ctas;
    if (cap > 0 && ctas > (uint32_t)cap) ctas = (uint32_t)cap;
    if (pair) ctas *= 2;

    plan.pub.kernel = split3 ? srtMatmulKernelTcgen05Split : pair ? srtMatmulKernelTcgen05Pair : srtMatmulKernelTcgen05;
    plan.pub.tileM = (int32_t)tile_m; plan.pub.tileN = (int32_t)bn; plan.pub.tileK = (int32_t)kb_elems;
    plan.pub.stages = (int32_t)stages;
    plan.pub.ctas = (int32_t)ctas;
    plan.pub.tiles = (int32_t)tiles;
    plan.pub.swapped = plan.swapped;
    plan.pub.aMajor = plan.ta.mn_major; plan.pub.bMajor = plan.tb.mn_major;
    plan.pub.fp32Split = split3;
    plan.pub.splitK = (int32_t)splits;
    plan.pub.workspaceBytes = splits > 1 ? (size_t)splits * Q.batch * Q.M * Q.N * 4 : 0;
    plan.pub.dynamicSmemBytes = (size_t)stages * stage_bytes + kEpilogueStagingBytes + 1024;
    // the transposed plan of a row-major result needs the reduce pass to place the elements
    return !skinny_swap || (plan.pub.kernel == srtMatmulKernelTcgen05 && splits > 1);
}

void make_plan(const Problem& P, const DeviceInfo& dev, Plan& plan)
{
    // A few rows against a wide operand (a small batch through a Dense layer): as given, the rows
    // occupy a fraction of the MMA's 128 and every 64 columns cost a whole tile.  Transposed, the
    // wide dimension is tiled 128 at a time and the rows are the MMA's N (64): half the MMA
    // instructions per unit of work at the same number of units.
    const Choice choice = effective_choice(P);
    const bool untuned = choice.force == 0 && choice.tile_n == 0 && choice.stages == 0 && choice.max_ctas == 0 && choice.split_k == 0;
    if (untuned && dev.sm100 && P.type != real32F && P.batch == 1 && P.M >= 1 && P.M <= kSkinnyRows && P.N >= 512 && P.K >= 1024 &&
        P.o_n == 1 && make_plan_impl(P, dev, plan, true))
        return;
    make_plan_impl(P, dev, plan, false);
}

// ------------------------------------------------------------------ tensor maps
cudaError_t encode_operand(CUtensorMap* map, const Problem& Q, const char* ptr, const TcOperand& t, uint64_t rows,
                           long long s_b, uint32_t box_rows, OperandParams& op)
{
    const uint32_t elem = Q.elem;
    const uint32_t kb_elems = kRowBytes / elem;
    const bool bcast = (Q.batch == 1 || s_b == 0);
    CUtensorMapDataType dt = Q.type == real32F ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                             : Q.type == real16F ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    cuuint64_t gdim[3], gstride[2];
    cuuint32_t box[3], estr[3] = {1, 1, 1};
    if (!t.mn_major) {
        gdim[0] = Q.K; gdim[1] = rows;
        box[0] = kb_elems; box[1] = box_rows;
        op.chunks = 1; op.chunk_elems = box_rows; op.chunk_bytes = box_rows * kRowBytes;
        // rows of 128 bytes, groups of 8 rows 1024 bytes apart; the leading offset is unused
        op.desc_lo_fixed = 1u << 16;
        op.kstep = 32 >> 4;                       // next 32 bytes of K inside the swizzled row
    } else {
        gdim[0] = rows; gdim[1] = Q.K;
        box[0] = kb_elems; box[1] = kb_elems;     // 128 bytes of M/N by one stage of K
        op.chunks = box_rows / kb_elems; op.chunk_elems = kb_elems; op.chunk_bytes = kb_elems * kRowBytes;
        // 128 bytes of M/N per row, one row per k; 8-row groups 1024 bytes apart (stride
        // offset), the next 128 bytes of M/N one chunk further (leading offset)
        op.desc_lo_fixed = ((op.chunk_bytes >> 4) & 0x3fffu) << 16;
        op.kstep = ((32 / elem) * kRowBytes) >> 4;  // one MMA consumes 32/elem rows of k
    }
    op.mn_major = t.mn_major;
    op.batch_mul = bcast ? 0 : 1;
    // stride offset 1024 bytes, descriptor version 1 (bit 46), 128-byte swizzle (bits 61-63 = 2)
    op.desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);
    CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B;
    if (t.mn_major && elem == 4) {
        // M/N-contiguous 32-bit operands exist in one shared-memory layout only: 128-byte rows
        // swizzled in 32-byte units (layout type 1), whose pattern repeats every 4 rows (512 bytes)
        op.desc_hi = (512u >> 4) | (1u << 14) | (1u << 29);
        swizzle = CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B;
    }
    gdim[2] = bcast ? 1 : Q.batch;
    gstride[0] = (cuuint64_t)t.ld * elem;
    gstride[1] = bcast ? gstride[0] * gdim[1] : (cuuint64_t)s_b * elem;
    box[2] = 1;
    CUresult r = g_encode(map, dt, 3, const_cast<char*>(ptr), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(cudaErrorInvalidValue, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return cudaSuccess;
}

// Opt-in to large dynamic shared memory once per (kernel instantiation, device); `done` is a
// per-instantiation bit mask of devices.
template <typename Kernel>
cudaError_t ensure_smem_attr(Kernel kernel, std::atomic<uint64_t>& done, size_t smem)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const uint64_t bit = 1ull << (dev & 63);
    if (done.load(std::memory_order_acquire) & bit) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 1024);
    (void)smem;
    if (e != cudaSuccess) return e;
    done.fetch_or(bit, std::memory_order_release);
    return cudaSuccess;
}

template <typename T, uint32_t BN, typename OutT = T, bool GATHER = false>
cudaError_t launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, const GemmParams& gp, uint32_t ctas, size_t smem,
                      cudaStream_t stream, const typename PeerArgOf<GATHER>::type& peers = typename PeerArgOf<GATHER>::type())
{
    auto kernel = gemm_tcgen05_kernel<T, BN, OutT, GATHER>;
    static std::atomic<uint64_t> attr_done{0};
    cudaError_t e = ensure_smem_attr(kernel, attr_done, smem);
    if (e != cudaSuccess) return e;
    kernel<<<ctas, kGemmThreads, smem, stream>>>(ma, mb, mo, gp, peers);
    return cudaGetLastError();
}

// The gathering form of the one-CTA kernel.
template <typename T>
cudaError_t launch_tc_gather_bn(uint32_t bn, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, const GemmParams& gp,
                                uint32_t ctas, size_t smem, cudaStream_t stream, const PeerMaps& peers)
{
    switch (bn) {
    case 64: return launch_tc<T, 64, T, true>(ma, mb, mo, gp, ctas, smem, stream, peers);
    case 128: return launch_tc<T, 128, T, true>(ma, mb, mo, gp, ctas, smem, stream, peers);
    default: return launch_tc<T, 256, T, true>(ma, mb, mo, gp, ctas, smem, stream, peers);
    }
}

template <typename T, typename OutT = T>
cudaError_t launch_tc_bn(uint32_t bn, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, const GemmParams& gp, uint32_t ctas,
                         size_t smem, cudaStream_t stream)
{
    switch (bn) {
    case 64: return launch_tc<T, 64, OutT>(ma, mb, mo, gp, ctas, smem, stream);
    case 128: return launch_tc<T, 128, OutT>(ma, mb, mo, gp, ctas, smem, stream);
    default: return launch_tc<T, 256, OutT>(ma, mb, mo, gp, ctas, smem, stream);
    }
}

template <uint32_t BN>
cudaError_t launch_split(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, const GemmParams& gp, uint32_t ctas, size_t smem,
                         cudaStream_t stream)
{
    auto kernel = gemm_tcgen05_split_kernel<BN>;
    static std::atomic<uint64_t> attr_done{0};
    cudaError_t e = ensure_smem_attr(kernel, attr_done, smem);
    if (e != cudaSuccess) return e;
    kernel<<<ctas, kSplitThreads, smem, stream>>>(ma, mb, mo, gp);
    return cudaGetLastError();
}

template <typename T, uint32_t BN, bool GATHER = false>
cudaError_t launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, const GemmParams& gp, uint32_t ctas, size_t smem,
                        cudaStream_t stream, const typename PeerArgOf<GATHER>::type& peers = typename PeerArgOf<GATHER>::type())
{
    auto kernel = gemm_tcgen05_pair_kernel<T, BN, GATHER>;
    static std::atomic<uint64_t> attr_done{0};
    static std::atomic<int> cluster_cache[64];           // max co-resident pairs per device, 0 = unknown
    cudaError_t e = ensure_smem_attr(kernel, attr_done, smem);
    if (e != cudaSuccess) return e;
    int dev = 0;
    e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3(ctas, 1, 1);
    cfg.blockDim = dim3(kGemmThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // SMs that cannot be paired inside their GPC stay idle: never ask for more pairs than fit at once
    int max_clusters = cluster_cache[dev & 63].load(std::memory_order_acquire);
    if (max_clusters == 0) {
        // queried once, with the largest shared-memory footprint the kernel may be launched with
        cudaLaunchConfig_t q = cfg;
        q.dynamicSmemBytes = 227 * 1024 - 1024;
        e = cudaOccupancyMaxActiveClusters(&max_clusters, kernel, &q);
        if (e != cudaSuccess) return e;
        if (max_clusters < 1) return cudaErrorLaunchOutOfResources;
        cluster_cache[dev & 63].store(max_clusters, std::memory_order_release);
    }
    if (ctas / 2 > (uint32_t)max_clusters) cfg.gridDim.x = 2u * (uint32_t)max_clusters;
    return cudaLaunchKernelEx(&cfg, kernel, ma, mb, mo, gp, peers);
}

template <typename T>
cudaError_t launch_pair_bn(uint32_t bn, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, const GemmParams& gp,
                           uint32_t ctas, size_t smem, cudaStream_t stream)
{
    if (bn == 128) return launch_pair<T, 128>(ma, mb, mo, gp, ctas, smem, stream);
    return launch_pair<T, 256>(ma, mb, mo, gp, ctas, smem, stream);
}

// The gathering form of the pair kernel (product + stores of every tile to the peers' buffers).
template <typename T>
cudaError_t launch_pair_gather_bn(uint32_t bn, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, const GemmParams& gp,
                                  uint32_t ctas, size_t smem, cudaStream_t stream, const PeerMaps& peers)
{
    if (bn == 128) return launch_pair<T, 128, true>(ma, mb, mo, gp, ctas, smem, stream, peers);
    return launch_pair<T, 256, true>(ma, mb, mo, gp, ctas, smem, stream, peers);
}

// Everything a launch needs, computed once per distinct call signature (see the call cache).
struct Prepared {
    int32_t kernel = srtMatmulKernelNone;
    srtDataType type = real32F;
    uint32_t bn = 0, ctas = 0;
    size_t smem = 0;
    CUtensorMap ma, mb, mo;
    GemmParams gp;
    SimtParams sp;
    dim3 grid;
    uint32_t simt_tile = kSimtTile;
    // split-K only
    uint32_t splits = 1;
    size_t ws_bytes = 0;
    void* ws_bound = nullptr;        // workspace the output tensor map and gp.out currently point at
    bool static_scratch = false;     // split-K partial sums go to the library's static array (srtMatmulNoAlloc)
    ReduceParams rp;
    // TF32 + BFloat16-correction pair kernel only: the packed op(b) lives in the workspace
    CUtensorMap mbc;
    X3Params xp;
    PackParams pk;
    uint32_t reduce_vec = 1, reduce_blocks = 0;
};

// Tensor map of an output view for the epilogue's bulk stores: boxes of 32 rows x 128 bytes,
// 128-byte swizzle.  `base` is the view's first element (the caller's buffer, or the same view
// in a peer's buffer).  False when the view is not TMA-addressable.
bool encode_out_map(CUtensorMap* map, const Problem& Q, long long ldo, void* base)
{
    const CUtensorMapDataType dt = Q.type == real32F ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                   : Q.type == real16F ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                       : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const bool one = Q.batch == 1;
    cuuint64_t gdim[3] = {Q.N, Q.M, one ? 1 : Q.batch};
    cuuint64_t gstride[2] = {(cuuint64_t)ldo * Q.elem, one ? (cuuint64_t)ldo * Q.elem * Q.M : (cuuint64_t)Q.o_b * Q.elem};
    cuuint32_t box[3] = {kRowBytes / Q.elem, 32, 1}, estr[3] = {1, 1, 1};
    if (reinterpret_cast<uintptr_t>(base) % 16 != 0) return false;
    return gstride[1] % 16 == 0 && gstride[0] < (1ull << 40) && gstride[1] < (1ull << 40) &&
           g_encode(map, dt, 3, base, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

cudaError_t prepare_tc(const Plan& plan, Prepared& pr)
{
    const Problem& Q = plan.Q;
    const bool pair = plan.pub.kernel == srtMatmulKernelTcgen05Pair;
    const uint32_t bn = (uint32_t)plan.pub.tileN;
    const uint32_t tile_m = (uint32_t)plan.pub.tileM;
    const uint32_t b_rows = pair ? bn / 2 : bn;           // rows of B each CTA stages
    GemmParams& gp = pr.gp;
    memset(&gp, 0, sizeof gp);
    cudaError_t e = encode_operand(&pr.ma, Q, Q.a, plan.ta, Q.M, Q.a_b, kTileM, gp.a);
    if (e != cudaSuccess) return e;
    e = encode_operand(&pr.mb, Q, Q.b, plan.tb, Q.N, Q.b_b, b_rows, gp.b);
    if (e != cudaSuccess) return e;

    gp.M = (uint32_t)Q.M; gp.N = (uint32_t)Q.N; gp.K = (uint32_t)Q.K; gp.batch = (uint32_t)Q.batch;
    gp.tiles_m = (uint32_t)((Q.M + tile_m - 1) / tile_m);
    gp.tiles_n = (uint32_t)((Q.N + bn - 1) / bn);
    gp.tiles_per_batch = gp.tiles_m * gp.tiles_n;
    gp.tiles_total = (uint32_t)plan.pub.tiles;
    gp.k_splits = plan.splits;
    gp.num_tiles = gp.tiles_total * plan.splits;          // work units
    gp.kb_elems = kRowBytes / Q.elem;
    gp.k_blocks = (uint32_t)((Q.K + gp.kb_elems - 1) / gp.kb_elems);
    gp.kb_per_split = plan.splits > 1 ? plan.kb_per_split : gp.k_blocks;
    gp.group_m = pair ? 8 : 16;                           // 2048 rows of A per group either way
    set_tile_walk(gp);
    gp.stages = (uint32_t)plan.pub.stages;
    gp.stage_tx_bytes = kATileBytes + b_rows * kRowBytes;
    // instruction descriptor: fp32 accumulator, input format, majorness, N >> 3, M >> 4
    const uint32_t fmt = Q.type == real16F ? 0u : Q.type == real16BF ? 1u : 2u;
    gp.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)plan.ta.mn_major << 15) |
               ((uint32_t)plan.tb.mn_major << 16) | ((bn >> 3) << 17) | ((tile_m >> 4) << 24);
    gp.out = Q.out;
    gp.ldo = Q.N == 1 ? (Q.M == 1 ? 1 : Q.o_m) : (Q.M == 1 ? (long long)Q.N : Q.o_m);
    gp.out_batch_stride = Q.o_b;
    gp.bias = Q.bias;
    gp.bias_stride = Q.bias_stride;
    gp.bias_mode = plan.bias_mode;
    gp.act = Q.act;
    gp.out_vec_ok = (reinterpret_cast<uintptr_t>(Q.out) % 16 == 0) && ((gp.ldo * (long long)Q.elem) % 16 == 0) &&
                    ((Q.o_b * (long long)Q.elem) % 16 == 0) && (Q.N > 1 ? Q.o_n == 1 : true);
    // bulk tensor stores need the same alignment as 16-byte vector stores
    gp.out_tma = 0;
    memset(&pr.mo, 0, sizeof pr.mo);
    if (gp.out_vec_ok && Q.N > 1 && encode_out_map(&pr.mo, Q, gp.ldo, Q.out)) gp.out_tma = 1;
    pr.kernel = plan.pub.kernel;
    pr.type = Q.type;
    pr.bn = bn;
    pr.smem = plan.pub.dynamicSmemBytes;
    pr.ctas = (uint32_t)plan.pub.ctas;
    pr.splits = plan.splits;
    pr.ws_bytes = 0;
    pr.ws_bound = nullptr;
    pr.static_scratch = false;
    if (plan.splits > 1) {
        // first pass: raw fp32 partial sums into the workspace (bound at launch); bias,
        // activation, rounding and the output view belong to the reduce pass
        pr.ws_bytes = plan.pub.workspaceBytes;
        ReduceParams& rp = pr.rp;
        memset(&rp, 0, sizeof rp);
        rp.splits = plan.splits;
        rp.slice = (unsigned long long)Q.batch * Q.M * Q.N;
        rp.M = (uint32_t)Q.M; rp.N = (uint32_t)Q.N; rp.batch = (uint32_t)Q.batch;
        rp.out = Q.out;
        rp.o_b = Q.o_b; rp.o_m = Q.o_m; rp.o_n = Q.o_n;
        rp.bias = Q.bias; rp.bias_stride = Q.bias_stride; rp.bias_mode = plan.bias_mode; rp.act = Q.act;
        pr.reduce_vec = (Q.N % 4 == 0) ? 4 : 1;
        const unsigned long long groups = rp.slice / pr.reduce_vec;
        unsigned long long blocks = (groups + 255) / 256;
        if (blocks > 148ull * 16) blocks = 148ull * 16;
        pr.reduce_blocks = (uint32_t)blocks;
        gp.out = nullptr;
        gp.ldo = (long long)Q.N;
        gp.out_batch_stride = (long long)(Q.M * Q.N);
        gp.bias = nullptr; gp.bias_mode = 0; gp.act = kActIdentity;
        gp.out_vec_ok = (Q.N % 4 == 0);
        gp.out_tma = 0;
    }
    return cudaSuccess;
}

// Points a split-K launch at its workspace: the partial-sum kernel's output pointer and
// output tensor map, and the reduce pass' input.
cudaError_t bind_workspace(Prepared& pr, void* ws)
{
    GemmParams& gp = pr.gp;
    gp.out = ws;
    pr.rp.ws = static_cast<const float*>(ws);
    gp.out_tma = 0;
    if (gp.out_vec_ok && gp.N > 1) {
        cuuint64_t gdim[3] = {gp.N, gp.M, (cuuint64_t)gp.batch * pr.splits};
        cuuint64_t gstride[2] = {(cuuint64_t)gp.N * 4, (cuuint64_t)gp.M * gp.N * 4};
        cuuint32_t box[3] = {32, 32, 1}, estr[3] = {1, 1, 1};
        if (g_encode(&pr.mo, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, ws, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS)
            gp.out_tma = 1;
    }
    pr.ws_bound = ws;
    return cudaSuccess;
}

// ------------------------------------------------------------------ TF32 + BFloat16-correction pair kernel
cudaError_t prepare_x3(const Plan& plan, Prepared& pr)
{
    const Problem& Q = plan.Q;
    X3Params& xp = pr.xp;
    memset(&xp, 0, sizeof xp);
    GemmParams& gp = xp.g;
    cudaError_t e = encode_operand(&pr.ma, Q, Q.a, plan.ta, Q.M, Q.a_b, kTileM, gp.a);
    if (e != cudaSuccess) return e;
    gp.b = gp.a;                                          // the packed op(b) is K-contiguous too
    gp.b.batch_mul = (Q.batch == 1 || Q.b_b == 0) ? 0 : 1;
    gp.M = (uint32_t)Q.M; gp.N = (uint32_t)Q.N; gp.K = (uint32_t)Q.K; gp.batch = (uint32_t)Q.batch;
    const uint32_t bn = (uint32_t)plan.pub.tileN;
    gp.tiles_m = (uint32_t)((Q.M + 255) / 256);
    gp.tiles_n = (uint32_t)((Q.N + bn - 1) / bn);
    gp.tiles_per_batch = gp.tiles_m * gp.tiles_n;
    gp.tiles_total = (uint32_t)plan.pub.tiles;
    gp.k_splits = 1;
    gp.num_tiles = gp.tiles_total;
    gp.kb_elems = 32;
    gp.k_blocks = (uint32_t)((Q.K + 31) / 32);
    gp.kb_per_split = gp.k_blocks;
    gp.group_m = 8;
    set_tile_walk(gp);
    gp.stages = (uint32_t)plan.pub.stages;
    gp.stage_tx_bytes = 0;
    // instruction descriptors: fp32 accumulator, both operands K-major, N = tile width, M = 256
    const uint32_t shape = (1u << 4) | ((bn >> 3) << 17) | ((256u >> 4) << 24);
    xp.idesc_tf32 = shape | (2u << 7) | (2u << 10);
    xp.idesc_bf16 = shape | (1u << 7) | (1u << 10);
    gp.out = Q.out;
    gp.ldo = Q.N == 1 ? (Q.M == 1 ? 1 : Q.o_m) : (Q.M == 1 ? (long long)Q.N : Q.o_m);
    gp.out_batch_stride = Q.o_b;
    gp.bias = Q.bias;
    gp.bias_stride = Q.bias_stride;
    gp.bias_mode = plan.bias_mode;
    gp.act = Q.act;
    gp.out_vec_ok = (reinterpret_cast<uintptr_t>(Q.out) % 16 == 0) && ((gp.ldo * (long long)Q.elem) % 16 == 0) &&
                    ((Q.o_b * (long long)Q.elem) % 16 == 0) && (Q.N > 1 ? Q.o_n == 1 : true);
    gp.out_tma = 0;
    memset(&pr.mo, 0, sizeof pr.mo);
    if (gp.out_vec_ok && Q.N > 1 && encode_out_map(&pr.mo, Q, gp.ldo, Q.out)) gp.out_tma = 1;
    PackParams& pk = pr.pk;
    memset(&pk, 0, sizeof pk);
    pk.b = reinterpret_cast<const float*>(Q.b);
    pk.b_b = gp.b.batch_mul ? Q.b_b : 0; pk.b_n = Q.b_n; pk.b_k = Q.b_k;
    pk.N = (uint32_t)Q.N; pk.K = (uint32_t)Q.K; pk.Kp = gp.k_blocks * 32; pk.batch = gp.b.batch_mul ? (uint32_t)Q.batch : 1u;
    pr.kernel = srtMatmulKernelTf32x3Pair;
    pr.type = Q.type;
    pr.bn = bn;
    pr.smem = plan.pub.dynamicSmemBytes;
    pr.ctas = (uint32_t)plan.pub.ctas;
    pr.splits = 1;
    pr.ws_bytes = plan.pub.workspaceBytes;
    pr.ws_bound = nullptr;
    pr.static_scratch = false;
    return cudaSuccess;
}

// Points the pack pass and the tensor maps of the packed op(b) at the workspace: Bh = fp32 [items][N][Kp],
// then Bc = bf16 [items][N][2 Kp].  Rows beyond N are never written: the maps end at N and TMA zero-fills.
cudaError_t bind_pack(Prepared& pr, void* ws)
{
    PackParams& pk = pr.pk;
    const uint64_t rows = (uint64_t)pk.batch * pk.N;
    pk.bh = static_cast<float*>(ws);
    pk.bc = reinterpret_cast<__nv_bfloat16*>(static_cast<char*>(ws) + rows * pk.Kp * 4);
    {
        cuuint64_t gdim[3] = {pk.Kp, pk.N, pk.batch};
        cuuint64_t gstride[2] = {(cuuint64_t)pk.Kp * 4, (cuuint64_t)pk.Kp * 4 * pk.N};
        cuuint32_t box[3] = {32, pr.bn / 2, 1}, estr[3] = {1, 1, 1};
        if (g_encode(&pr.mb, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, pk.bh, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return fail(cudaErrorInvalidValue, "cuTensorMapEncodeTiled failed for the packed fp32 operand");
    }
    {
        cuuint64_t gdim[3] = {2ull * pk.Kp, pk.N, pk.batch};
        cuuint64_t gstride[2] = {(cuuint64_t)pk.Kp * 4, (cuuint64_t)pk.Kp * 4 * pk.N};
        cuuint32_t box[3] = {64, pr.bn / 2, 1}, estr[3] = {1, 1, 1};
        if (g_encode(&pr.mbc, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, pk.bc, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return fail(cudaErrorInvalidValue, "cuTensorMapEncodeTiled failed for the packed correction operand");
    }
    pr.ws_bound = ws;
    return cudaSuccess;
}

template <uint32_t BN>
cudaError_t launch_x3_bn(const Prepared& pr, cudaStream_t stream)
{
    auto kernel = gemm_tf32x3_pair_kernel<BN>;
    static std::atomic<uint64_t> attr_done{0};
    static std::atomic<int> cluster_cache[64];
    cudaError_t e = ensure_smem_attr(kernel, attr_done, pr.smem);
    if (e != cudaSuccess) return e;
    int dev = 0;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return e;
    const PackParams& pk = pr.pk;
    const unsigned long long items = (unsigned long long)pk.batch * pk.N * (pk.Kp / 4);
    unsigned long long blocks = (items + 255) / 256;
    if (blocks > 148ull * 8) blocks = 148ull * 8;
    tf32x3_pack_kernel<<<(unsigned)blocks, 256, 0, stream>>>(pk);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    g_launches.fetch_add(1, std::memory_order_relaxed);
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3(pr.ctas, 1, 1);
    cfg.blockDim = dim3(x3_threads(BN), 1, 1);
    cfg.dynamicSmemBytes = pr.smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // scheduled while the pack pass still runs; the producer waits (griddepcontrol.wait) before its first load
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    int max_clusters = cluster_cache[dev & 63].load(std::memory_order_acquire);
    if (max_clusters == 0) {
        cudaLaunchConfig_t q = cfg;
        q.numAttrs = 1;
        q.dynamicSmemBytes = 227 * 1024 - 1024;
        e = cudaOccupancyMaxActiveClusters(&max_clusters, kernel, &q);
        if (e != cudaSuccess) return e;
        if (max_clusters < 1) return cudaErrorLaunchOutOfResources;
        cluster_cache[dev & 63].store(max_clusters, std::memory_order_release);
    }
    if (pr.ctas / 2 > (uint32_t)max_clusters) cfg.gridDim.x = 2u * (uint32_t)max_clusters;
    return cudaLaunchKernelEx(&cfg, kernel, pr.ma, pr.mb, pr.mbc, pr.mo, pr.xp);
}

cudaError_t launch_x3(const Prepared& pr, cudaStream_t stream)
{
    return pr.bn == 256 ? launch_x3_bn<256>(pr, stream) : launch_x3_bn<128>(pr, stream);
}

// Workspaces of split-K launches: one buffer per (device, stream), grown on demand.  Kernels of
// one stream run in order, so a stream never races with itself.  `slot` separates buffers that are
// alive at the same time on one stream (slot 0: split-K partial sums and column-sum partials;
// slot 1: the recurrent cells' gate input and fused product).
//
// Growth never waits for the GPU: the new buffer is allocated beside the old one and the old one is
// freed in stream order (cudaFreeAsync on the same stream, behind the kernels that still use it).
// A buffer that was handed out while its stream was being captured is baked into a CUDA graph that
// may be replayed at any later time: it is marked `captured` and, when a later call on the same
// stream handle needs more, it is kept alive (moved to the retained list) instead of freed.
// srtMatmulReleaseWorkspaces gives the memory back.
struct Workspace { int device; cudaStream_t stream; int slot; void* ptr; size_t bytes; bool captured; };
struct Retained { int device; void* ptr; bool captured; };
std::mutex g_ws_mutex;
std::vector<Workspace> g_workspaces;
std::vector<Retained> g_retained;

cudaError_t workspace_for(int device, cudaStream_t stream, size_t bytes, void** out, int slot = 0)
{
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess) {
        cap = cudaStreamCaptureStatusNone;
        (void)cudaGetLastError();
    }
    const bool capturing = cap != cudaStreamCaptureStatusNone;
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    Workspace* w = nullptr;
    for (Workspace& c : g_workspaces)
        if (c.device == device && c.stream == stream && c.slot == slot) { w = &c; break; }
    if (!w) {
        g_workspaces.push_back(Workspace{device, stream, slot, nullptr, 0, false});
        w = &g_workspaces.back();
    }
    if (w->bytes < bytes) {
        if (capturing)
            return fail(cudaErrorStreamCaptureUnsupported,
                        "the workspace of this stream would have to grow (%zu -> %zu bytes) during stream capture; run the same "
                        "call once before capturing", w->bytes, bytes);
        void* fresh = nullptr;
        cudaError_t e = cudaMalloc(&fresh, bytes);
        if (e != cudaSuccess) return fail(e, "cudaMalloc of a %zu-byte workspace failed: %s", bytes, cudaGetErrorString(e));
        if (w->ptr) {
            if (w->captured) {
                g_retained.push_back(Retained{device, w->ptr, true});
            } else if (cudaFreeAsync(w->ptr, stream) != cudaSuccess) {
                (void)cudaGetLastError();
                g_retained.push_back(Retained{device, w->ptr, false});       // freed by srtMatmulReleaseWorkspaces
            }
        }
        w->ptr = fresh;
        w->bytes = bytes;
        w->captured = false;
    }
    if (capturing) w->captured = true;
    *out = w->ptr;
    return cudaSuccess;
}

// ------------------------------------------------------------------ static scratch (srtMatmulNoAlloc)
// Part of the library image: every device that loads the library carries these 16 MiB from then
// until the process ends, whether or not the entry point is ever called.  In host code the name is
// only a handle for cudaGetSymbolAddress; the device address it yields is what the kernels receive.
constexpr size_t kNoAllocScratchBytes = 16u << 20;
static __device__ __align__(256) unsigned char g_no_alloc_scratch[kNoAllocScratchBytes];

std::mutex g_no_alloc_mutex;
void* g_no_alloc_ptr[64] = {};

// Device address of the scratch array on device `dev` (which must be current), looked up once per device.
cudaError_t no_alloc_scratch(int dev, void** out)
{
    std::lock_guard<std::mutex> lock(g_no_alloc_mutex);
    if (dev < 0 || dev >= 64) return fail(cudaErrorInvalidDevice, "device ordinal %d out of range", dev);
    if (!g_no_alloc_ptr[dev]) {
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_no_alloc_scratch);
        if (e != cudaSuccess) return fail(e, "cudaGetSymbolAddress of the static scratch failed: %s", cudaGetErrorString(e));
        g_no_alloc_ptr[dev] = ptr;
    }
    *out = g_no_alloc_ptr[dev];
    return cudaSuccess;
}

cudaError_t prepare_simt(const Plan& plan, Prepared& pr)
{
    const Problem& P = plan.Q;
    SimtParams& sp = pr.sp;
    memset(&sp, 0, sizeof sp);
    sp.M = (uint32_t)P.M; sp.N = (uint32_t)P.N; sp.K = (uint32_t)P.K; sp.batch = (uint32_t)P.batch;
    sp.a = P.a; sp.b = P.b; sp.out = P.out; sp.bias = P.bias;
    sp.a_b = P.a_b; sp.a_m = P.a_m; sp.a_k = P.a_k;
    sp.b_b = P.b_b; sp.b_k = P.b_k; sp.b_n = P.b_n;
    sp.o_b = P.o_b; sp.o_m = P.o_m; sp.o_n = P.o_n;
    sp.bias_stride = P.bias_stride;
    sp.has_bias = P.bias != nullptr;
    sp.act = P.act;
    sp.a_k_fast = (P.a_k == 1) || (P.a_m != 1);
    sp.b_n_fast = (P.b_n == 1) || (P.b_k != 1);
    const uint32_t st = (uint32_t)plan.pub.tileM;
    pr.simt_tile = st;
    const uint64_t tm = (P.M + st - 1) / st, tn = (P.N + st - 1) / st;
    if (tm > 65535) return fail(cudaErrorNotSupported, "strided kernel: more than 65535 row tiles");
    pr.grid = dim3((unsigned)tn, (unsigned)tm, (unsigned)P.batch);
    pr.kernel = srtMatmulKernelSimt;
    pr.type = P.type;
    // `pr` may be a recycled call-cache slot that last held a split-K launch
    pr.splits = 1;
    pr.ws_bytes = 0;
    pr.ws_bound = nullptr;
    pr.static_scratch = false;
    return cudaSuccess;
}

template <typename T, int VEC>
cudaError_t launch_reduce_as_dependent(const ReduceParams& rp, unsigned blocks, cudaStream_t stream)
{
    // programmatic dependent launch: the reduce grid is scheduled while the partial-sum kernel still
    // runs and waits inside the kernel (grid_dependency_wait) for its completion
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3(blocks, 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, splitk_reduce_kernel<T, VEC>, rp);
}

template <typename T>
cudaError_t launch_reduce_transposed(const ReduceParams& rp, cudaStream_t stream)
{
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3((rp.N + 31) / 32, (rp.M + 31) / 32, rp.batch);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, splitk_reduce_transposed_kernel<T>, rp);
}

cudaError_t launch_reduce(const Prepared& pr, cudaStream_t stream)
{
    const ReduceParams& rp = pr.rp;
    // output contiguous along M: reduce through a shared-memory transpose (grid.y and grid.z limits permitting)
    if (rp.o_m == 1 && rp.o_n != 1 && rp.M > 1 && (rp.M + 31) / 32 <= 65535 && rp.batch <= 65535) {
        switch (pr.type) {
        case real32F: return launch_reduce_transposed<float>(rp, stream);
        case real16F: return launch_reduce_transposed<__half>(rp, stream);
        default: return launch_reduce_transposed<__nv_bfloat16>(rp, stream);
        }
    }
    const unsigned blocks = pr.reduce_blocks;
    const bool v4 = pr.reduce_vec == 4;
    switch (pr.type) {
    case real32F: return v4 ? launch_reduce_as_dependent<float, 4>(rp, blocks, stream) : launch_reduce_as_dependent<float, 1>(rp, blocks, stream);
    case real16F: return v4 ? launch_reduce_as_dependent<__half, 4>(rp, blocks, stream) : launch_reduce_as_dependent<__half, 1>(rp, blocks, stream);
    default: return v4 ? launch_reduce_as_dependent<__nv_bfloat16, 4>(rp, blocks, stream)
                       : launch_reduce_as_dependent<__nv_bfloat16, 1>(rp, blocks, stream);
    }
}

cudaError_t launch_prepared(Prepared& pr, cudaStream_t stream)
{
    cudaError_t e;
    const uint32_t bn = pr.bn;
    // nanoseconds -> SM cycles at an upper bound of 2 cycles per nanosecond
    pr.gp.wait_cycles = pr.xp.g.wait_cycles = g_wait_limit_ns.load(std::memory_order_relaxed) * 2;
    if (pr.ws_bytes > 0) {
        int dev = 0;
        e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        void* ws = nullptr;
        e = pr.static_scratch ? no_alloc_scratch(dev, &ws) : workspace_for(dev, stream, pr.ws_bytes, &ws);
        if (e != cudaSuccess) return e;
        if (ws != pr.ws_bound) {
            e = pr.kernel == srtMatmulKernelTf32x3Pair ? bind_pack(pr, ws) : bind_workspace(pr, ws);
            if (e != cudaSuccess) return e;
        }
    }
    switch (pr.kernel) {
    case srtMatmulKernelTf32x3Pair:
        e = launch_x3(pr, stream);
        break;
    case srtMatmulKernelSimt:
        switch (pr.type) {
        case real32F:
            if (pr.simt_tile == 32) gemm_simt_kernel<float, 32><<<pr.grid, 256, 0, stream>>>(pr.sp);
            else                    gemm_simt_kernel<float, 64><<<pr.grid, 256, 0, stream>>>(pr.sp);
            break;
        case real16F:
            if (pr.simt_tile == 32) gemm_simt_kernel<__half, 32><<<pr.grid, 256, 0, stream>>>(pr.sp);
            else                    gemm_simt_kernel<__half, 64><<<pr.grid, 256, 0, stream>>>(pr.sp);
            break;
        default:
            if (pr.simt_tile == 32) gemm_simt_kernel<__nv_bfloat16, 32><<<pr.grid, 256, 0, stream>>>(pr.sp);
            else                    gemm_simt_kernel<__nv_bfloat16, 64><<<pr.grid, 256, 0, stream>>>(pr.sp);
            break;
        }
        e = cudaGetLastError();
        break;
    case srtMatmulKernelTcgen05Split:
        e = bn == 64    ? launch_split<64>(pr.ma, pr.mb, pr.mo, pr.gp, pr.ctas, pr.smem, stream)
            : bn == 128 ? launch_split<128>(pr.ma, pr.mb, pr.mo, pr.gp, pr.ctas, pr.smem, stream)
                        : launch_split<256>(pr.ma, pr.mb, pr.mo, pr.gp, pr.ctas, pr.smem, stream);
        break;
    case srtMatmulKernelTcgen05Pair:
        switch (pr.type) {
        case real32F: e = launch_pair_bn<float>(bn, pr.ma, pr.mb, pr.mo, pr.gp, pr.ctas, pr.smem, stream); break;
        case real16F: e = launch_pair_bn<__half>(bn, pr.ma, pr.mb, pr.mo, pr.gp, pr.ctas, pr.smem, stream); break;
        default: e = launch_pair_bn<__nv_bfloat16>(bn, pr.ma, pr.mb, pr.mo, pr.gp, pr.ctas, pr.smem, stream); break;
        }
        break;
    default:
        if (pr.splits > 1) {
            switch (pr.type) {
            case real32F: e = launch_tc_bn<float, float>(bn, pr.ma, pr.mb, pr.mo, pr.gp, pr.ctas, pr.smem, stream); break;
            case real16F: e = launch_tc_bn<__half, float>(bn, pr.ma, pr.mb, pr.mo, pr.gp, pr.ctas, pr.smem, stream); break;
            default: e = launch_tc_bn<__nv_bfloat16, float>(bn, pr.ma, pr.mb, pr.mo, pr.gp, pr.ctas, pr.smem, stream); break;
            }
        } else {
            switch (pr.type) {
            case real32F: e = launch_tc_bn<float>(bn, pr.ma, pr.mb, pr.mo, pr.gp, pr.ctas, pr.smem, stream); break;
            case real16F: e = launch_tc_bn<__half>(bn, pr.ma, pr.mb, pr.mo, pr.gp, pr.ctas, pr.smem, stream); break;
            default: e = launch_tc_bn<__nv_bfloat16>(bn, pr.ma, pr.mb, pr.mo, pr.gp, pr.ctas, pr.smem, stream); break;
            }
        }
        break;
    }
    if (e != cudaSuccess) return e;
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (pr.splits > 1) {
        e = launch_reduce(pr, stream);
        if (e == cudaSuccess) g_launches.fetch_add(1, std::memory_order_relaxed);
    }
    return e;
}

cudaError_t prepare_any(const Plan& plan, Prepared& pr)
{
    switch (plan.pub.kernel) {
    case srtMatmulKernelSimt: return prepare_simt(plan, pr);
    case srtMatmulKernelTf32x3Pair: return prepare_x3(plan, pr);
    default: return prepare_tc(plan, pr);
    }
}

// ------------------------------------------------------------------ call cache
// Repeated calls with the same pointers, geometry and options (a training loop, a benchmark,
// a layer applied to the same buffers) skip planning and tensor-map encoding.  The cache is
// per host thread -- a SwiftRT queue is used by one thread only -- so it needs no lock.
struct CallKey {
    Problem P;
    int32_t force, tile_n, stages, max_ctas, split_k;
    int32_t device;
    uint32_t plan_epoch;
    uint32_t no_alloc;              // 1: srtMatmulNoAlloc (split-K scratch = the static array)
};

constexpr int kCallCacheSize = 64;
struct CallCache {
    bool valid[kCallCacheSize] = {};
    CallKey key[kCallCacheSize];
    Prepared value[kCallCacheSize];
};
thread_local std::unique_ptr<CallCache> t_cache;

uint64_t hash_key(const CallKey& k)
{
    const unsigned char* p = reinterpret_cast<const unsigned char*>(&k);
    uint64_t h = 1469598103934665603ull;
    for (size_t i = 0; i < sizeof k; ++i) h = (h ^ p[i]) * 1099511628211ull;
    return h;
}

cudaError_t plan_for(const Problem& P, Plan& plan)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    DeviceInfo info;
    e = device_info(dev, info);
    if (e != cudaSuccess) return e;
    if (!info.sm100) return fail(cudaErrorNotSupported, "this library is built for sm_100a devices only");
    make_plan(P, info, plan);
    return cudaSuccess;
}

// ------------------------------------------------------------------ srtBiasActivationBackward
struct View3 { uint64_t batch, M, N; long long s_b, s_m, s_n; };

// rank 2 [M x N] or rank 3 [batch x M x N] descriptor -> sizes and element strides
cudaError_t view3(const srtTensorDescriptor* d, const char* what, View3& v)
{
    if (!d || !d->shape || !d->strides) return fail(cudaErrorInvalidValue, "%s: missing descriptor", what);
    if (d->rank != 2 && d->rank != 3) return fail(cudaErrorNotSupported, "%s must have rank 2 or 3", what);
    const uint32_t q = d->rank - 2;
    v.batch = d->rank == 3 ? d->shape[0] : 1;
    v.M = d->shape[q]; v.N = d->shape[q + 1];
    v.s_b = d->rank == 3 ? (long long)d->strides[0] : 0;
    v.s_m = (long long)d->strides[q]; v.s_n = (long long)d->strides[q + 1];
    return cudaSuccess;
}

template <typename T>
cudaError_t launch_dense_backward(const DenseBackwardParams& bp, bool vec, uint32_t chunks, void* dbias, long long dbias_stride,
                                  cudaStream_t stream)
{
    constexpr int kVec = 16 / sizeof(T);
    if (vec) {
        dim3 grid((bp.N + 32 * kVec - 1) / (32 * kVec), chunks, 1);
        dense_backward_kernel<T, kVec><<<grid, 256, 0, stream>>>(bp);
    } else {
        dim3 grid((bp.N + 31) / 32, chunks, 1);
        dense_backward_kernel<T, 1><<<grid, 256, 0, stream>>>(bp);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (dbias) {
        dense_backward_finish_kernel<T><<<(bp.N + 255) / 256, 256, 0, stream>>>(bp.partial, chunks, bp.N, static_cast<T*>(dbias),
                                                                                 dbias_stride);
        e = cudaGetLastError();
        if (e == cudaSuccess) g_launches.fetch_add(1, std::memory_order_relaxed);
    }
    return e;
}

// ------------------------------------------------------------------ plan table: file form and tuner
// One text line per entry:
//   type flags M N K batch  force tileN stages maxCtas splitK  microseconds
// under a header line.  Lines that do not parse are skipped.
constexpr const char* kPlanFileHeader = "srt_matmul_plan_cache v1";

int plan_table_load(const char* path)
{
    FILE* f = fopen(path, "r");
    if (!f) return -1;
    char line[512];
    int loaded = 0;
    bool header_ok = false;
    while (fgets(line, sizeof line, f)) {
        if (!header_ok) {
            if (strncmp(line, kPlanFileHeader, strlen(kPlanFileHeader)) != 0) { fclose(f); return -2; }
            header_ok = true;
            continue;
        }
        if (line[0] == '#' || line[0] == '\n') continue;
        PlanKey k;
        memset(&k, 0, sizeof k);
        Choice c;
        float us = 0.0f;
        unsigned long long M, N, K, batch;
        if (sscanf(line, "%d %u %llu %llu %llu %llu %d %d %d %d %d %f", &k.type, &k.flags, &M, &N, &K, &batch, &c.force, &c.tile_n,
                   &c.stages, &c.max_ctas, &c.split_k, &us) != 12)
            continue;
        if (c.force < 0 || c.force > srtMatmulKernelTf32x3Pair) continue;
        k.M = M; k.N = N; k.K = K; k.batch = batch;
        plan_store(k, c, us);
        ++loaded;
    }
    fclose(f);
    if (!header_ok) return -2;
    g_plan_epoch.fetch_add(1, std::memory_order_relaxed);
    return loaded;
}

int plan_table_save(const char* path)
{
    FILE* f = fopen(path, "w");
    if (!f) return -1;
    fprintf(f, "%s\n# type flags M N K batch  force tileN stages maxCtas splitK  microseconds\n", kPlanFileHeader);
    std::lock_guard<std::mutex> lock(g_plan_mutex);
    for (const PlanEntry& e : g_plan_table)
        fprintf(f, "%d %u %llu %llu %llu %llu %d %d %d %d %d %.3f\n", e.key.type, e.key.flags, (unsigned long long)e.key.M,
                (unsigned long long)e.key.N, (unsigned long long)e.key.K, (unsigned long long)e.key.batch, e.choice.force,
                e.choice.tile_n, e.choice.stages, e.choice.max_ctas, e.choice.split_k, e.us);
    const int n = (int)g_plan_table.size();
    fclose(f);
    return n;
}

// Average device time of one launch of `pr` on `stream`, in microseconds (events on that stream).
cudaError_t time_prepared(Prepared& pr, cudaStream_t stream, cudaEvent_t e0, cudaEvent_t e1, float& us)
{
    cudaError_t e = launch_prepared(pr, stream);               // warm-up: attributes, workspace, caches
    if (e != cudaSuccess) return e;
    if ((e = cudaEventRecord(e0, stream)) != cudaSuccess) return e;
    if ((e = launch_prepared(pr, stream)) != cudaSuccess) return e;
    if ((e = cudaEventRecord(e1, stream)) != cudaSuccess) return e;
    if ((e = cudaEventSynchronize(e1)) != cudaSuccess) return e;
    float ms = 0.0f;
    if ((e = cudaEventElapsedTime(&ms, e0, e1)) != cudaSuccess) return e;
    // as many repetitions as fit in ~10 ms, between 3 and 50
    int reps = ms > 0.0f ? (int)(10.0f / ms) : 50;
    if (reps < 3) reps = 3;
    if (reps > 50) reps = 50;
    if ((e = cudaEventRecord(e0, stream)) != cudaSuccess) return e;
    for (int i = 0; i < reps; ++i)
        if ((e = launch_prepared(pr, stream)) != cudaSuccess) return e;
    if ((e = cudaEventRecord(e1, stream)) != cudaSuccess) return e;
    if ((e = cudaEventSynchronize(e1)) != cudaSuccess) return e;
    if ((e = cudaEventElapsedTime(&ms, e0, e1)) != cudaSuccess) return e;
    us = ms * 1000.0f / (float)reps;
    return cudaSuccess;
}

// ------------------------------------------------------------------ srtLstmCell helpers
cudaError_t view2(const srtTensorDescriptor* d, const char* what, srtDataType type, uint64_t& rows, uint64_t& cols,
                         long long& s_m, long long& s_n)
{
    if (!d || !d->shape || !d->strides) return fail(cudaErrorInvalidValue, "srtLstmCell: %s: missing descriptor", what);
    if (d->rank != 2) return fail(cudaErrorInvalidValue, "srtLstmCell: %s must have rank 2", what);
    if (d->type != type) return fail(cudaErrorInvalidValue, "srtLstmCell: %s has a different element type", what);
    rows = d->shape[0]; cols = d->shape[1];
    s_m = (long long)d->strides[0]; s_n = (long long)d->strides[1];
    return cudaSuccess;
}

inline bool aligned16(const void* p, long long row_stride_elems, size_t elem)
{
    return reinterpret_cast<uintptr_t>(p) % 16 == 0 && (row_stride_elems * (long long)elem) % 16 == 0;
}

template <typename T>
cudaError_t launch_lstm_elementwise(const ConcatParams* cp, const LstmGateParams* gp, cudaStream_t stream)
{
    constexpr int kVec = 16 / sizeof(T);
    if (cp) {
        const bool vec = cp->x_n == 1 && cp->h_n == 1 && cp->nx % kVec == 0 && cp->nh % kVec == 0 &&
                         aligned16(cp->x, cp->x_m, sizeof(T)) && aligned16(cp->h, cp->h_m, sizeof(T));
        unsigned blocks = cp->rows < 148u * 16 ? cp->rows : 148u * 16;
        if (vec) concat_kernel<T, kVec><<<blocks, 256, 0, stream>>>(*cp);
        else     concat_kernel<T, 1><<<blocks, 256, 0, stream>>>(*cp);
    } else {
        const bool vec = gp->hidden % kVec == 0 && gp->c_n == 1 && gp->nc_n == 1 && gp->nh_n == 1 &&
                         aligned16(gp->cell, gp->c_m, sizeof(T)) && aligned16(gp->new_cell, gp->nc_m, sizeof(T)) &&
                         aligned16(gp->new_hidden, gp->nh_m, sizeof(T));
        const uint32_t hchunks = vec ? gp->hidden / kVec : gp->hidden;
        const uint32_t rows_per_pass = 256 / (hchunks < 256 ? hchunks : 256);
        unsigned long long groups = ((unsigned long long)gp->rows + rows_per_pass - 1) / rows_per_pass;
        unsigned blocks = (unsigned)(groups < 148ull * 16 ? groups : 148ull * 16);
        if (vec) lstm_gates_kernel<T, kVec><<<blocks, 256, 0, stream>>>(*gp);
        else     lstm_gates_kernel<T, 1><<<blocks, 256, 0, stream>>>(*gp);
    }
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) g_launches.fetch_add(1, std::memory_order_relaxed);
    return e;
}

// ------------------------------------------------------------------ driver entry points for multicast buffers
struct DriverApi {
    CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags) = nullptr;
    CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*) = nullptr;
    CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
    CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long) = nullptr;
    CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
    CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
    CUresult (*MemRelease)(CUmemGenericAllocationHandle) = nullptr;
    CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
    CUresult (*MemAddressFree)(CUdeviceptr, size_t) = nullptr;
    CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
    CUresult (*MemUnmap)(CUdeviceptr, size_t) = nullptr;
    CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
    CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
    bool ok = false;
};

template <typename F>
bool driver_symbol(const char* name, F& fn)
{
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) return false;
    fn = reinterpret_cast<F>(p);
    return true;
}

const DriverApi& driver_api()
{
    static DriverApi api = [] {
        DriverApi d;
        d.ok = driver_symbol("cuMulticastGetGranularity", d.MulticastGetGranularity) && driver_symbol("cuMulticastCreate", d.MulticastCreate) &&
               driver_symbol("cuMulticastAddDevice", d.MulticastAddDevice) && driver_symbol("cuMulticastBindMem", d.MulticastBindMem) &&
               driver_symbol("cuMulticastUnbind", d.MulticastUnbind) && driver_symbol("cuMemCreate", d.MemCreate) &&
               driver_symbol("cuMemRelease", d.MemRelease) && driver_symbol("cuMemAddressReserve", d.MemAddressReserve) &&
               driver_symbol("cuMemAddressFree", d.MemAddressFree) && driver_symbol("cuMemMap", d.MemMap) &&
               driver_symbol("cuMemUnmap", d.MemUnmap) && driver_symbol("cuMemSetAccess", d.MemSetAccess) &&
               driver_symbol("cuDeviceGetAttribute", d.DeviceGetAttribute);
        return d;
    }();
    return api;
}

struct MulticastBuffer {
    int n = 0;
    int devices[kMaxPeers + 1] = {};
    size_t size = 0;
    CUmemGenericAllocationHandle mc = 0;
    CUmemGenericAllocationHandle mem[kMaxPeers + 1] = {};
    CUdeviceptr va[kMaxPeers + 1] = {};
    CUdeviceptr mc_va = 0;
    bool bound[kMaxPeers + 1] = {};
};

void multicast_destroy(MulticastBuffer* b)
{
    const DriverApi& d = driver_api();
    for (int i = 0; i < b->n; ++i) {
        cudaSetDevice(b->devices[i]);
        cudaDeviceSynchronize();
    }
    if (b->mc_va) { d.MemUnmap(b->mc_va, b->size); d.MemAddressFree(b->mc_va, b->size); }
    for (int i = 0; i < b->n; ++i) {
        if (b->va[i]) { d.MemUnmap(b->va[i], b->size); d.MemAddressFree(b->va[i], b->size); }
        if (b->bound[i]) d.MulticastUnbind(b->mc, b->devices[i], 0, b->size);
        if (b->mem[i]) d.MemRelease(b->mem[i]);
    }
    if (b->mc) d.MemRelease(b->mc);
    delete b;
}


// ------------------------------------------------------------------ one product
// Parses, plans (or finds the prepared launch of an identical earlier call) and enqueues.
// `no_alloc`: split-K partial sums go to the static scratch array; products whose partial sums do
// not fit there are refused before anything is launched.
cudaError_t run_matmul(const void* a, const srtTensorDescriptor* aDesc, bool transA, const void* b,
                       const srtTensorDescriptor* bDesc, bool transB, const void* bias,
                       const srtTensorDescriptor* biasDesc, srtActivationType activation, void* out,
                       const srtTensorDescriptor* oDesc, cudaStream_t stream, bool no_alloc)
{
    CallKey key;
    memset(&key, 0, sizeof key);                 // padding bytes are part of the hashed key
    Problem& P = key.P;
    cudaError_t e = parse(a, aDesc, transA, b, bDesc, transB, bias, biasDesc, (int)activation, out, oDesc, P);
    if (e != cudaSuccess) return e;
    if (is_empty(P)) return cudaSuccess;
    DeviceScope scope(stream);
    if (scope.status != cudaSuccess) return scope.status;
    key.force = g_tuning.force_kernel.load(std::memory_order_relaxed);
    key.tile_n = g_tuning.tile_n.load(std::memory_order_relaxed);
    key.stages = g_tuning.stages.load(std::memory_order_relaxed);
    key.max_ctas = g_tuning.max_ctas.load(std::memory_order_relaxed);
    key.split_k = g_tuning.split_k.load(std::memory_order_relaxed);
    key.device = scope.device;
    key.plan_epoch = g_plan_epoch.load(std::memory_order_relaxed);
    key.no_alloc = no_alloc ? 1u : 0u;
    if (!t_cache) t_cache.reset(new CallCache());
    const int slot = (int)(hash_key(key) % kCallCacheSize);
    if (t_cache->valid[slot] && memcmp(&t_cache->key[slot], &key, sizeof key) == 0)
        return launch_prepared(t_cache->value[slot], stream);

    Plan plan;
    e = plan_for(P, plan);
    if (e != cudaSuccess) return e;
    if (no_alloc && plan.pub.workspaceBytes > kNoAllocScratchBytes) {
        if (plan.splits > 1)
            return fail(cudaErrorInvalidValue,
                        "srtMatmulNoAlloc: this product needs %zu bytes of scratch (%u partial results of %llu x %llu x %llu "
                        "fp32 values) but the static scratch holds %zu; use srtMatmul, or srtMatmulSetSplitK(1)",
                        (size_t)plan.pub.workspaceBytes, plan.splits, (unsigned long long)plan.Q.batch,
                        (unsigned long long)plan.Q.M, (unsigned long long)plan.Q.N, kNoAllocScratchBytes);
        return fail(cudaErrorInvalidValue,
                    "srtMatmulNoAlloc: this product needs %zu bytes of scratch (the pre-split copy of its %llu x %llu operand) but the "
                    "static scratch holds %zu; use srtMatmul, or srtMatmulSetTuning(srtMatmulKernelTcgen05Split, 0, 0, 0)",
                    (size_t)plan.pub.workspaceBytes, (unsigned long long)plan.Q.N, (unsigned long long)plan.Q.K, kNoAllocScratchBytes);
    }
    Prepared& pr = t_cache->value[slot];
    t_cache->valid[slot] = false;
    e = prepare_any(plan, pr);
    if (e != cudaSuccess) return e;
    pr.static_scratch = no_alloc && pr.ws_bytes > 0;
    e = launch_prepared(pr, stream);
    if (e == cudaSuccess) {
        t_cache->key[slot] = key;
        t_cache->valid[slot] = true;
    }
    return e;
}

}  // namespace

// ===================================================================== exported entry points
extern "C" {

cudaError_t srtMatmulBiasActivation(const void* a, const srtTensorDescriptor* aDesc, bool transA, const void* b,
                                    const srtTensorDescriptor* bDesc, bool transB, const void* bias,
                                    const srtTensorDescriptor* biasDesc, srtActivationType activation, void* out,
                                    const srtTensorDescriptor* oDesc, cudaStream_t stream)
{
    return run_matmul(a, aDesc, transA, b, bDesc, transB, bias, biasDesc, activation, out, oDesc, stream, false);
}

cudaError_t srtMatmul(const void* a, const srtTensorDescriptor* aDesc, bool transA, const void* b,
                      const srtTensorDescriptor* bDesc, bool transB, void* out, const srtTensorDescriptor* oDesc,
                      cudaStream_t stream)
{
    return srtMatmulBiasActivation(a, aDesc, transA, b, bDesc, transB, nullptr, nullptr, srtActivationIdentity, out,
                                   oDesc, stream);
}

cudaError_t srtMatmulQueryPlan(const void* a, const srtTensorDescriptor* aDesc, bool transA, const void* b,
                               const srtTensorDescriptor* bDesc, bool transB, const void* out,
                               const srtTensorDescriptor* oDesc, srtMatmulPlan* plan_out)
{
    if (!plan_out) return fail(cudaErrorInvalidValue, "null plan");
    Problem P;
    cudaError_t e = parse(a, aDesc, transA, b, bDesc, transB, nullptr, nullptr, srtActivationIdentity, out, oDesc, P);
    if (e != cudaSuccess) return e;
    if (is_empty(P)) { memset(plan_out, 0, sizeof *plan_out); return cudaSuccess; }      // nothing to launch
    Plan plan;
    e = plan_for(P, plan);
    if (e != cudaSuccess) return e;
    *plan_out = plan.pub;
    return cudaSuccess;
}

cudaError_t srtMatmulSetTuning(int32_t forceKernel, int32_t tileN, int32_t stages, int32_t maxCtas)
{
    if (forceKernel < 0 || forceKernel > srtMatmulKernelTf32x3Pair) return fail(cudaErrorInvalidValue, "unknown kernel id");
    if (tileN != 0 && tileN != 64 && tileN != 128 && tileN != 256) return fail(cudaErrorInvalidValue, "tileN must be 0, 64, 128 or 256");
    if (stages != 0 && (stages < 2 || stages > 8)) return fail(cudaErrorInvalidValue, "stages must be 0 or 2..8");
    if (maxCtas < 0) return fail(cudaErrorInvalidValue, "maxCtas must be >= 0");
    g_tuning.force_kernel = forceKernel;
    g_tuning.tile_n = tileN;
    g_tuning.stages = stages;
    g_tuning.max_ctas = maxCtas;
    return cudaSuccess;
}

cudaError_t srtMatmulSetSplitK(int32_t splits)
{
    if (splits < 0 || splits > 64) return fail(cudaErrorInvalidValue, "splits must be 0 (automatic) or 1..64");
    g_tuning.split_k = splits;
    return cudaSuccess;
}

cudaError_t srtMatmulTune(const void* a, const srtTensorDescriptor* aDesc, bool transA, const void* b,
                          const srtTensorDescriptor* bDesc, bool transB, const void* bias,
                          const srtTensorDescriptor* biasDesc, srtActivationType activation, void* out,
                          const srtTensorDescriptor* oDesc, cudaStream_t stream, srtMatmulPlan* best, float* bestMicroseconds)
{
    Problem P;
    memset(&P, 0, sizeof P);
    cudaError_t e = parse(a, aDesc, transA, b, bDesc, transB, bias, biasDesc, (int)activation, out, oDesc, P);
    if (e != cudaSuccess) return e;
    if (is_empty(P)) return fail(cudaErrorInvalidValue, "srtMatmulTune: empty result");
    DeviceScope scope(stream);
    if (scope.status != cudaSuccess) return scope.status;
    // candidates: the cost model's own choice first, then every kernel / tile width the type allows
    std::vector<Choice> cands;
    cands.push_back(Choice{0, 0, 0, 0, 0});
    if (P.type == real32F) {
        cands.push_back(Choice{srtMatmulKernelSimt, 0, 0, 0, 0});
        for (int32_t tn : {64, 128, 256}) cands.push_back(Choice{srtMatmulKernelTcgen05Split, tn, 0, 0, 0});
        cands.push_back(Choice{srtMatmulKernelTf32x3Pair, 0, 0, 0, 0});
    } else {
        for (int32_t tn : {64, 128, 256}) {
            cands.push_back(Choice{srtMatmulKernelTcgen05, tn, 0, 0, 0});
            // the same without split-K and with fixed numbers of parts (few tiles, long reductions)
            for (int32_t sk : {1, 2, 4, 8, 16}) cands.push_back(Choice{srtMatmulKernelTcgen05, tn, 0, 0, sk});
        }
        for (int32_t tn : {128, 256}) cands.push_back(Choice{srtMatmulKernelTcgen05Pair, tn, 0, 0, 0});
    }
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if ((e = cudaEventCreate(&e0)) != cudaSuccess) return e;
    if ((e = cudaEventCreate(&e1)) != cudaSuccess) { cudaEventDestroy(e0); return e; }
    std::vector<srtMatmulPlan> seen;
    float best_us = 0.0f;
    Choice best_choice = cands[0];
    srtMatmulPlan best_plan;
    memset(&best_plan, 0, sizeof best_plan);
    bool have = false;
    Prepared* pr = new Prepared();
    for (const Choice& c : cands) {
        t_choice_override = &c;
        Plan plan;
        e = plan_for(P, plan);
        t_choice_override = nullptr;
        if (e != cudaSuccess) break;
        bool dup = false;
        for (const srtMatmulPlan& s : seen) dup = dup || memcmp(&s, &plan.pub, sizeof s) == 0;
        if (dup) continue;
        seen.push_back(plan.pub);
        e = prepare_any(plan, *pr);
        if (e != cudaSuccess) break;
        float us = 0.0f;
        e = time_prepared(*pr, stream, e0, e1, us);
        if (e != cudaSuccess) break;
        if (!have || us < best_us) { have = true; best_us = us; best_choice = c; best_plan = plan.pub; }
    }
    delete pr;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (e != cudaSuccess) return e;
    if (!have) return fail(cudaErrorUnknown, "srtMatmulTune: no candidate ran");
    // pin what the winner actually ran, so that a later change of the cost model cannot alter it
    best_choice.force = best_plan.kernel;
    if (best_plan.kernel != srtMatmulKernelSimt) {
        best_choice.tile_n = best_plan.tileN;
        best_choice.stages = best_plan.stages;
        if (best_choice.split_k == 0 && best_plan.splitK <= 1) best_choice.split_k = 1;
    }
    plan_store(plan_key(P), best_choice, best_us);
    g_plan_epoch.fetch_add(1, std::memory_order_relaxed);
    if (best) *best = best_plan;
    if (bestMicroseconds) *bestMicroseconds = best_us;
    // leave `out` holding the product computed by the chosen plan
    return srtMatmulBiasActivation(a, aDesc, transA, b, bDesc, transB, bias, biasDesc, activation, out, oDesc, stream);
}

cudaError_t srtMatmulPlanCacheSave(const char* path)
{
    if (!path) return fail(cudaErrorInvalidValue, "srtMatmulPlanCacheSave: null path");
    return plan_table_save(path) >= 0 ? cudaSuccess : fail(cudaErrorInvalidValue, "srtMatmulPlanCacheSave: cannot write %s", path);
}

cudaError_t srtMatmulPlanCacheLoad(const char* path, int32_t* entries)
{
    if (!path) return fail(cudaErrorInvalidValue, "srtMatmulPlanCacheLoad: null path");
    const int n = plan_table_load(path);
    if (n == -1) return fail(cudaErrorInvalidValue, "srtMatmulPlanCacheLoad: cannot read %s", path);
    if (n == -2) return fail(cudaErrorInvalidValue, "srtMatmulPlanCacheLoad: %s is not a plan cache file", path);
    if (entries) *entries = n;
    return cudaSuccess;
}

cudaError_t srtMatmulPlanCacheClear(void)
{
    {
        std::lock_guard<std::mutex> lock(g_plan_mutex);
        g_plan_table.clear();
    }
    g_plan_epoch.fetch_add(1, std::memory_order_relaxed);
    return cudaSuccess;
}

cudaError_t srtMatmulCheckStatus(cudaStream_t stream, uint32_t* status)
{
    if (!status) return fail(cudaErrorInvalidValue, "null status");
    DeviceScope scope(stream);
    if (scope.status != cudaSuccess) return scope.status;
    cudaError_t e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return e;
    uint32_t v = 0;
    e = cudaMemcpyFromSymbol(&v, srt::g_gemm_status, sizeof v);
    if (e != cudaSuccess) return e;
    if (v != 0) {
        const uint32_t zero = 0;
        e = cudaMemcpyToSymbol(srt::g_gemm_status, &zero, sizeof zero);
        if (e != cudaSuccess) return e;
    }
    *status = v;
    return cudaSuccess;
}

cudaError_t srtBiasActivationBackward(const void* dy, const srtTensorDescriptor* dyDesc, const void* y,
                                      const srtTensorDescriptor* yDesc, srtActivationType activation, void* dz,
                                      const srtTensorDescriptor* dzDesc, void* dbias, const srtTensorDescriptor* dbiasDesc,
                                      cudaStream_t stream)
{
    if (!dy || !dyDesc) return fail(cudaErrorInvalidValue, "null dy");
    if (!dz && !dbias) return fail(cudaErrorInvalidValue, "nothing to compute: dz and dbias are both null");
    View3 vg, vy{}, vz{};
    cudaError_t e = view3(dyDesc, "dy", vg);
    if (e != cudaSuccess) return e;
    const srtDataType type = dyDesc->type;
    const uint32_t elem = elem_size(type);
    if (elem == 0) return fail(cudaErrorNotSupported, "element type %d is not computed by this library", (int)type);
    switch ((int)activation) {
    case srtActivationIdentity: case srtActivationRelu: case srtActivationSigmoid: case srtActivationTanh: break;
    case srtActivationGelu: case srtActivationGeluTanh: break;       // `y` carries the pre-activation values
    case srtActivationClippedRelu: case srtActivationElu:
        return fail(cudaErrorNotSupported, "clippedRelu and elu need coefficients that this entry point does not carry");
    default: return fail(cudaErrorInvalidValue, "unknown activation %d", (int)activation);
    }
    const bool need_y = activation != srtActivationIdentity;
    if (need_y) {
        if (!y) return fail(cudaErrorInvalidValue, "the forward output y (the pre-activation values for gelu) is needed for this activation's derivative");
        e = view3(yDesc, "y", vy);
        if (e != cudaSuccess) return e;
        if (yDesc->type != type || vy.batch != vg.batch || vy.M != vg.M || vy.N != vg.N)
            return fail(cudaErrorInvalidValue, "y must have the type and shape of dy");
    }
    if (dz) {
        e = view3(dzDesc, "dz", vz);
        if (e != cudaSuccess) return e;
        if (dzDesc->type != type || vz.batch != vg.batch || vz.M != vg.M || vz.N != vg.N)
            return fail(cudaErrorInvalidValue, "dz must have the type and shape of dy");
    }
    long long dbias_stride = 1;
    if (dbias) {
        if (!dbiasDesc || !dbiasDesc->shape || !dbiasDesc->strides || dbiasDesc->rank != 1 || dbiasDesc->shape[0] != vg.N ||
            dbiasDesc->type != type)
            return fail(cudaErrorInvalidValue, "dbias must be rank 1 with %llu elements of dy's type", (unsigned long long)vg.N);
        dbias_stride = (long long)dbiasDesc->strides[0];
    }
    if (vg.M == 0 || vg.N == 0 || vg.batch == 0 || vg.M > 0x7fffffffull || vg.N > 0x7fffffffull || vg.batch > 0x7fffffffull)
        return fail(cudaErrorInvalidValue, "dimension outside the supported range");
    g_error[0] = 0;
    DeviceScope scope(stream);
    if (scope.status != cudaSuccess) return scope.status;
    const int dev = scope.device;
    DeviceInfo info;
    e = device_info(dev, info);
    if (e != cudaSuccess) return e;

    DenseBackwardParams bp;
    memset(&bp, 0, sizeof bp);
    bp.dy = dy; bp.y = need_y ? y : nullptr; bp.dz = dz;
    bp.dy_b = vg.s_b; bp.dy_m = vg.s_m; bp.dy_n = vg.s_n;
    bp.y_b = vy.s_b; bp.y_m = vy.s_m; bp.y_n = vy.s_n;
    bp.dz_b = vz.s_b; bp.dz_m = vz.s_m; bp.dz_n = vz.s_n;
    bp.M = (uint32_t)vg.M; bp.N = (uint32_t)vg.N; bp.batch = (uint32_t)vg.batch;
    bp.act = (uint32_t)activation;
    const uint32_t vecw = 16 / elem;
    auto vec_ok = [&](const void* ptr, const View3& v) {
        return reinterpret_cast<uintptr_t>(ptr) % 16 == 0 && (v.s_n == 1 || v.N == 1) && (v.s_m * (long long)elem) % 16 == 0 &&
               (v.s_b * (long long)elem) % 16 == 0;
    };
    const bool vec = vg.N % vecw == 0 && vec_ok(dy, vg) && (!need_y || vec_ok(y, vy)) && (!dz || vec_ok(dz, vz));
    // enough blocks to fill the device a few times over, at least 8 rows (one per warp) per chunk
    const uint64_t rows = vg.batch * vg.M;
    const uint64_t col_blocks = (vg.N + 32 * (vec ? vecw : 1) - 1) / (32 * (vec ? vecw : 1));
    // one wave of 6 blocks per SM (40 registers x 256 threads): as many row loads in flight as fit
    uint64_t chunks = ((uint64_t)info.sms * 6) / col_blocks;
    if (chunks > (rows + 7) / 8) chunks = (rows + 7) / 8;
    if (chunks < 1) chunks = 1;
    if (chunks > 65535) chunks = 65535;
    bp.rows_per_chunk = (uint32_t)((rows + chunks - 1) / chunks);
    chunks = (rows + bp.rows_per_chunk - 1) / bp.rows_per_chunk;
    bp.partial = nullptr;
    if (dbias) {
        void* ws = nullptr;
        e = workspace_for(dev, stream, (size_t)chunks * vg.N * sizeof(float), &ws);
        if (e != cudaSuccess) return e;
        bp.partial = static_cast<float*>(ws);
    }
    switch (type) {
    case real32F: return launch_dense_backward<float>(bp, vec, (uint32_t)chunks, dbias, dbias_stride, stream);
    case real16F: return launch_dense_backward<__half>(bp, vec, (uint32_t)chunks, dbias, dbias_stride, stream);
    default: return launch_dense_backward<__nv_bfloat16>(bp, vec, (uint32_t)chunks, dbias, dbias_stride, stream);
    }
}

// ------------------------------------------------------------------ srtActivationForward
// ---------------------------------------------------------------------------------------------
// srtMatrixTransform and its layout helpers (cublaslt/MatrixTransform.swift:21-129, MatrixLayout.swift:21-204)
uint64_t srtMatrixLayoutLeadingDimension(srtOrder order, uint64_t rows, uint64_t cols)
{
    switch ((int)order) {
    case srtOrderRow: return cols;
    case srtOrderCol: return rows;
    case srtOrderColTiled32: return 32 * rows;
    case srtOrderColTiledTC32x32: return 32 * ((rows + 31) / 32 * 32);
    default: return 0;
    }
}

uint64_t srtMatrixLayoutElementCount(srtOrder order, uint64_t rows, uint64_t cols, uint64_t ld)
{
    if (rows == 0 || cols == 0) return 0;
    switch ((int)order) {
    case srtOrderRow: return (rows - 1) * ld + cols;
    case srtOrderCol: return (cols - 1) * ld + rows;
    case srtOrderColTiled32: return ((cols - 1) / 32) * ld + 32 * rows;
    case srtOrderColTiledTC32x32: return ((cols - 1) / 32) * ld + 32 * ((rows + 31) / 32 * 32);
    default: return 0;
    }
}

namespace {
cudaError_t check_layout(const srtMatrixLayout* l, const char* name)
{
    switch ((int)l->type) {
    case real32F: case real16F: case real16BF: case real8I: break;
    default: return fail(cudaErrorNotSupported, "srtMatrixTransform: element type %d of %s is not computed", (int)l->type, name);
    }
    switch ((int)l->order) {
    case srtOrderRow: case srtOrderCol: case srtOrderColTiled32: case srtOrderColTiledTC32x32: break;
    case srtOrderColTiledTC32x8:
        return fail(cudaErrorNotSupported, "srtMatrixTransform: order colTiledTC32x8 of %s is not computed (an operand layout of SM 7.2 / 7.5)", name);
    default: return fail(cudaErrorInvalidValue, "srtMatrixTransform: unknown order %d of %s", (int)l->order, name);
    }
    if (l->rows > 0x7fffffffull || l->cols > 0x7fffffffull)          // "only values that can be expressed as Int32" (MatrixLayout.swift:115-143)
        return fail(cudaErrorInvalidValue, "srtMatrixTransform: rows / cols of %s outside the Int32 range", name);
    if (l->batchCount < 1) return fail(cudaErrorInvalidValue, "srtMatrixTransform: batchCount of %s must be at least 1", name);
    if (l->leadingDimension < 0 || l->batchStride < 0)
        return fail(cudaErrorInvalidValue, "srtMatrixTransform: negative leading dimension or batch stride of %s", name);
    if (l->rows != 0 && l->cols != 0 &&
        (uint64_t)l->leadingDimension < srtMatrixLayoutLeadingDimension(l->order, l->rows, l->cols))
        return fail(cudaErrorInvalidValue, "srtMatrixTransform: leading dimension %lld of %s is below the %llu its order needs",
                    (long long)l->leadingDimension, name, (unsigned long long)srtMatrixLayoutLeadingDimension(l->order, l->rows, l->cols));
    return cudaSuccess;
}
}  // namespace

cudaError_t srtMatrixTransform(const float* alpha, const void* A, const srtMatrixLayout* aLayout, bool transA,
                               const float* beta, const void* B, const srtMatrixLayout* bLayout, bool transB,
                               void* C, const srtMatrixLayout* cLayout, cudaStream_t stream)
{
    if (!alpha || !A || !aLayout || !C || !cLayout) return fail(cudaErrorInvalidValue, "srtMatrixTransform: null alpha, A, C or layout");
    const float bt = beta ? *beta : 0.0f;
    const bool use_b = bt != 0.0f;
    if (use_b && (!B || !bLayout)) return fail(cudaErrorInvalidValue, "srtMatrixTransform: beta is not 0 but B or its layout is null");
    cudaError_t e = check_layout(aLayout, "A");
    if (e != cudaSuccess) return e;
    if ((e = check_layout(cLayout, "C")) != cudaSuccess) return e;
    if (use_b && (e = check_layout(bLayout, "B")) != cudaSuccess) return e;
    auto same_shape = [&](const srtMatrixLayout* l, bool t) {
        return (t ? l->cols : l->rows) == cLayout->rows && (t ? l->rows : l->cols) == cLayout->cols && l->batchCount == cLayout->batchCount;
    };
    if (!same_shape(aLayout, transA)) return fail(cudaErrorInvalidValue, "srtMatrixTransform: op(A) and C differ in rows, cols or batchCount");
    if (use_b && !same_shape(bLayout, transB)) return fail(cudaErrorInvalidValue, "srtMatrixTransform: op(B) and C differ in rows, cols or batchCount");
    if (cLayout->rows == 0 || cLayout->cols == 0) return cudaSuccess;
    g_error[0] = 0;
    DeviceScope scope(stream);
    if (scope.status != cudaSuccess) return scope.status;
    TransformParams tp;
    memset(&tp, 0, sizeof tp);
    auto fill = [](StoredMatrix& m, const void* ptr, const srtMatrixLayout* l, bool t) {
        m.ptr = const_cast<void*>(ptr);
        m.ld = l->leadingDimension;
        m.batch_stride = l->batchStride;
        m.order = (int32_t)l->order;
        m.type = (int32_t)l->type;
        m.transposed = t ? 1u : 0u;
    };
    fill(tp.a, A, aLayout, transA);
    fill(tp.c, C, cLayout, false);
    if (use_b) fill(tp.b, B, bLayout, transB); else tp.b = tp.a;
    tp.alpha = *alpha;
    tp.beta = bt;
    tp.use_b = use_b ? 1u : 0u;
    tp.rows = (uint32_t)cLayout->rows;
    tp.cols = (uint32_t)cLayout->cols;
    tp.batch = (uint32_t)cLayout->batchCount;
    tp.tiles_r = (tp.rows + kTransformTile - 1) / kTransformTile;
    tp.tiles_c = (tp.cols + kTransformTile - 1) / kTransformTile;
    // V elements per access: 16 bytes of the widest element type, if every operand's addresses allow it
    auto size_of = [](int32_t t) { return t == kTypeF32 ? 4u : t == kTypeI8 ? 1u : 2u; };
    uint32_t widest = size_of(tp.a.type) > size_of(tp.c.type) ? size_of(tp.a.type) : size_of(tp.c.type);
    if (use_b && size_of(tp.b.type) > widest) widest = size_of(tp.b.type);
    uint32_t narrowest = size_of(tp.a.type) < size_of(tp.c.type) ? size_of(tp.a.type) : size_of(tp.c.type);
    if (use_b && size_of(tp.b.type) < narrowest) narrowest = size_of(tp.b.type);
    auto aligned = [&](const StoredMatrix& m, uint32_t v) {
        return reinterpret_cast<uintptr_t>(m.ptr) % (v * size_of(m.type)) == 0 && m.ld % v == 0 && m.batch_stride % v == 0;
    };
    auto all_aligned = [&](uint32_t v) { return aligned(tp.a, v) && aligned(tp.c, v) && (!use_b || aligned(tp.b, v)); };
    // 16 bytes of the narrowest type per thread (wider operands then move as several 16-byte accesses), else 16 bytes
    // of the widest, else element by element
    uint32_t vec = 16 / narrowest;
    if (!all_aligned(vec)) vec = 16 / widest;
    if (!all_aligned(vec)) vec = 1;
    const bool stream_form = runs_along_columns(tp.a) == runs_along_columns(tp.c) &&
                             (!use_b || runs_along_columns(tp.b) == runs_along_columns(tp.c));
    if (stream_form) {
        const bool along_columns = runs_along_columns(tp.c);
        const unsigned long long fast = along_columns ? tp.cols : tp.rows, slow = along_columns ? tp.rows : tp.cols;
        const unsigned long long work = (unsigned long long)tp.batch * slow * ((fast + vec - 1) / vec);
        unsigned long long blocks = (work + kTransformThreads - 1) / kTransformThreads;
        if (blocks > 148ull * 16) blocks = 148ull * 16;
        const unsigned grid = (unsigned)blocks;
        const bool raw = !use_b && tp.alpha == 1.0f && tp.a.type == tp.c.type;
        switch (vec) {
        case 16:
            if (raw) matrix_transform_stream_kernel<16, true><<<grid, kTransformThreads, 0, stream>>>(tp);
            else     matrix_transform_stream_kernel<16, false><<<grid, kTransformThreads, 0, stream>>>(tp);
            break;
        case 8:
            if (raw) matrix_transform_stream_kernel<8, true><<<grid, kTransformThreads, 0, stream>>>(tp);
            else     matrix_transform_stream_kernel<8, false><<<grid, kTransformThreads, 0, stream>>>(tp);
            break;
        case 4:
            if (raw) matrix_transform_stream_kernel<4, true><<<grid, kTransformThreads, 0, stream>>>(tp);
            else     matrix_transform_stream_kernel<4, false><<<grid, kTransformThreads, 0, stream>>>(tp);
            break;
        default:
            if (raw) matrix_transform_stream_kernel<1, true><<<grid, kTransformThreads, 0, stream>>>(tp);
            else     matrix_transform_stream_kernel<1, false><<<grid, kTransformThreads, 0, stream>>>(tp);
            break;
        }
    } else if (!use_b && tp.alpha == 1.0f && tp.a.type == tp.c.type && widest <= 2 && vec == 16 / widest &&
               tp.rows % (widest == 1 ? 128u : 64u) == 0 && tp.cols % (widest == 1 ? 128u : 64u) == 0) {
        // a pure transposition of whole tiles of 1- or 2-byte elements: packed words, byte permutes
        const unsigned long long edge = widest == 1 ? 128 : 64;
        const unsigned long long tiles = (tp.rows / edge) * (tp.cols / edge) * tp.batch;
        const unsigned grid = (unsigned)(tiles < 148ull * 8 ? tiles : 148ull * 8);
        if (widest == 1) matrix_transform_transpose_kernel<1><<<grid, kTransformThreads, 0, stream>>>(tp);
        else             matrix_transform_transpose_kernel<2><<<grid, kTransformThreads, 0, stream>>>(tp);
    } else {
        const unsigned long long tiles = (unsigned long long)tp.tiles_r * tp.tiles_c * tp.batch;
        const unsigned grid = (unsigned)(tiles < 148ull * 8 ? tiles : 148ull * 8);
        switch (vec) {
        case 16: matrix_transform_tile_kernel<16><<<grid, kTransformThreads, 0, stream>>>(tp); break;
        case 8: matrix_transform_tile_kernel<8><<<grid, kTransformThreads, 0, stream>>>(tp); break;
        case 4: matrix_transform_tile_kernel<4><<<grid, kTransformThreads, 0, stream>>>(tp); break;
        default: matrix_transform_tile_kernel<1><<<grid, kTransformThreads, 0, stream>>>(tp); break;
        }
    }
    e = cudaGetLastError();
    if (e == cudaSuccess) g_launches.fetch_add(1, std::memory_order_relaxed);
    return e;
}

cudaError_t srtActivationForward(const void* z, const srtTensorDescriptor* zDesc, srtActivationType activation, void* y,
                                 const srtTensorDescriptor* yDesc, cudaStream_t stream)
{
    if (!z || !y || !zDesc || !yDesc) return fail(cudaErrorInvalidValue, "srtActivationForward: null tensor");
    View3 vz, vy;
    cudaError_t e = view3(zDesc, "z", vz);
    if (e != cudaSuccess) return e;
    if ((e = view3(yDesc, "y", vy)) != cudaSuccess) return e;
    const srtDataType type = zDesc->type;
    const uint32_t elem = elem_size(type);
    if (elem == 0) return fail(cudaErrorNotSupported, "element type %d is not computed by this library", (int)type);
    if (yDesc->type != type || vy.batch != vz.batch || vy.M != vz.M || vy.N != vz.N)
        return fail(cudaErrorInvalidValue, "y must have the type and shape of z");
    switch ((int)activation) {
    case srtActivationIdentity: case srtActivationRelu: case srtActivationSigmoid: case srtActivationTanh:
    case srtActivationGelu: case srtActivationGeluTanh: break;
    case srtActivationClippedRelu: case srtActivationElu:
        return fail(cudaErrorNotSupported, "clippedRelu and elu need coefficients that this entry point does not carry");
    default: return fail(cudaErrorInvalidValue, "unknown activation %d", (int)activation);
    }
    if (vz.M == 0 || vz.N == 0 || vz.batch == 0) return cudaSuccess;
    if (vz.M > 0x7fffffffull || vz.N > 0x7fffffffull || vz.batch > 0x7fffffffull)
        return fail(cudaErrorInvalidValue, "dimension outside the supported range");
    g_error[0] = 0;
    DeviceScope scope(stream);
    if (scope.status != cudaSuccess) return scope.status;
    DenseBackwardParams bp;
    memset(&bp, 0, sizeof bp);
    bp.dy = z; bp.dz = y;
    bp.dy_b = vz.s_b; bp.dy_m = vz.s_m; bp.dy_n = vz.s_n;
    bp.dz_b = vy.s_b; bp.dz_m = vy.s_m; bp.dz_n = vy.s_n;
    bp.M = (uint32_t)vz.M; bp.N = (uint32_t)vz.N; bp.batch = (uint32_t)vz.batch;
    bp.act = (uint32_t)activation;
    const uint32_t vecw = 16 / elem;
    auto vec_ok = [&](const void* ptr, const View3& v) {
        return reinterpret_cast<uintptr_t>(ptr) % 16 == 0 && (v.s_n == 1 || v.N == 1) && (v.s_m * (long long)elem) % 16 == 0 &&
               (v.s_b * (long long)elem) % 16 == 0;
    };
    const bool vec = vz.N % vecw == 0 && vec_ok(z, vz) && vec_ok(y, vy);
    const unsigned long long work = vz.batch * vz.M * ((vz.N + (vec ? vecw : 1) - 1) / (vec ? vecw : 1));
    unsigned long long blocks = (work + 255) / 256;
    if (blocks > 148ull * 16) blocks = 148ull * 16;
    const unsigned grid = (unsigned)blocks;
    switch (type) {
    case real32F:
        if (vec) activation_forward_kernel<float, 4><<<grid, 256, 0, stream>>>(bp);
        else     activation_forward_kernel<float, 1><<<grid, 256, 0, stream>>>(bp);
        break;
    case real16F:
        if (vec) activation_forward_kernel<__half, 8><<<grid, 256, 0, stream>>>(bp);
        else     activation_forward_kernel<__half, 1><<<grid, 256, 0, stream>>>(bp);
        break;
    default:
        if (vec) activation_forward_kernel<__nv_bfloat16, 8><<<grid, 256, 0, stream>>>(bp);
        else     activation_forward_kernel<__nv_bfloat16, 1><<<grid, 256, 0, stream>>>(bp);
        break;
    }
    e = cudaGetLastError();
    if (e == cudaSuccess) g_launches.fetch_add(1, std::memory_order_relaxed);
    return e;
}

// ------------------------------------------------------------------ srtMatmulReleaseWorkspaces
cudaError_t srtMatmulReleaseWorkspaces(bool includeCaptured)
{
    int cur = 0;
    cudaError_t e = cudaGetDevice(&cur);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    cudaError_t first = cudaSuccess;
    auto release = [&](int device, void* ptr) {
        cudaError_t r = cudaSetDevice(device);
        if (r == cudaSuccess) r = cudaDeviceSynchronize();      // nothing enqueued may still use the buffer
        if (r == cudaSuccess) r = cudaFree(ptr);
        if (r != cudaSuccess && first == cudaSuccess) first = r;
    };
    std::vector<Workspace> keep_ws;
    for (const Workspace& w : g_workspaces) {
        if (w.ptr && (includeCaptured || !w.captured)) release(w.device, w.ptr);
        else if (w.ptr) keep_ws.push_back(w);
    }
    g_workspaces.swap(keep_ws);
    std::vector<Retained> keep_rt;
    for (const Retained& r : g_retained) {
        if (includeCaptured || !r.captured) release(r.device, r.ptr);
        else keep_rt.push_back(r);
    }
    g_retained.swap(keep_rt);
    cudaSetDevice(cur);
    return first == cudaSuccess ? cudaSuccess : fail(first, "srtMatmulReleaseWorkspaces: %s", cudaGetErrorString(first));
}

// ------------------------------------------------------------------ srtLstmCell
cudaError_t srtLstmCell(const void* input, const srtTensorDescriptor* inputDesc, const void* hidden,
                        const srtTensorDescriptor* hiddenDesc, const void* cell, const srtTensorDescriptor* cellDesc,
                        const void* fusedWeight, const srtTensorDescriptor* weightDesc, const void* fusedBias,
                        const srtTensorDescriptor* biasDesc, void* newCell, const srtTensorDescriptor* newCellDesc,
                        void* newHidden, const srtTensorDescriptor* newHiddenDesc, cudaStream_t stream)
{
    if (!input || !cell || !fusedWeight || !newCell || !newHidden || !inputDesc)
        return fail(cudaErrorInvalidValue, "srtLstmCell: null tensor");
    const srtDataType type = inputDesc->type;
    if (type != real32F && type != real16F && type != real16BF)
        return fail(cudaErrorNotSupported, "srtLstmCell: element type %d is outside this library", (int)type);
    uint64_t rows, nx, r2, nh, r3, c3, wk, wn, r4, c4, r5, c5;
    long long x_m, x_n, h_m = 0, h_n = 0, c_m, c_n, w_m, w_n, nc_m, nc_n, nh_m, nh_n;
    cudaError_t e;
    if ((e = view2(inputDesc, "input", type, rows, nx, x_m, x_n)) != cudaSuccess) return e;
    // hidden == NULL: `input` is the gate input already, [batch x (inputSize + hiddenSize)], and nothing is concatenated
    const bool preconcatenated = hidden == nullptr;
    if (preconcatenated) {
        if ((e = view2(cellDesc, "cell", type, r2, nh, c_m, c_n)) != cudaSuccess) return e;
        if (nx < nh) return fail(cudaErrorInvalidValue, "srtLstmCell: a gate input has at least hiddenSize columns");
        nx -= nh;
    } else if ((e = view2(hiddenDesc, "hidden", type, r2, nh, h_m, h_n)) != cudaSuccess) {
        return e;
    }
    if ((e = view2(cellDesc, "cell", type, r3, c3, c_m, c_n)) != cudaSuccess) return e;
    if ((e = view2(weightDesc, "fusedWeight", type, wk, wn, w_m, w_n)) != cudaSuccess) return e;
    if ((e = view2(newCellDesc, "newCell", type, r4, c4, nc_m, nc_n)) != cudaSuccess) return e;
    if ((e = view2(newHiddenDesc, "newHidden", type, r5, c5, nh_m, nh_n)) != cudaSuccess) return e;
    if (r2 != rows || r3 != rows || r4 != rows || r5 != rows || c3 != nh || c4 != nh || c5 != nh)
        return fail(cudaErrorInvalidValue, "srtLstmCell: state tensors must be [batch x hiddenSize]");
    if (wk != nx + nh || wn != 4 * nh)
        return fail(cudaErrorInvalidValue, "srtLstmCell: fusedWeight must be [(inputSize + hiddenSize) x 4 hiddenSize], got %llu x %llu",
                    (unsigned long long)wk, (unsigned long long)wn);
    if (fusedBias && (!biasDesc || biasDesc->rank != 1 || biasDesc->shape[0] != 4 * nh || biasDesc->type != type))
        return fail(cudaErrorInvalidValue, "srtLstmCell: fusedBias must be rank 1 with 4 hiddenSize elements");
    if (rows == 0 || nh == 0) return cudaSuccess;
    if (rows > 0xffffffffull || nx + nh > 0xffffffffull || 4 * nh > 0xffffffffull)
        return fail(cudaErrorNotSupported, "srtLstmCell: extents beyond 32 bits");

    const size_t elem = type == real32F ? 4 : 2;
    // the gate input is staged in the workspace only when the library concatenates it
    const size_t gate_bytes = preconcatenated ? 0 : (((size_t)rows * (nx + nh) * elem + 255) & ~(size_t)255);
    const size_t fused_bytes = (size_t)rows * 4 * nh * elem;
    DeviceScope scope(stream);
    if (scope.status != cudaSuccess) return scope.status;
    const int dev = scope.device;
    void* ws = nullptr;
    if ((e = workspace_for(dev, stream, gate_bytes + fused_bytes, &ws, 1)) != cudaSuccess) return e;
    const void* gate_in = preconcatenated ? input : ws;
    void* fused = static_cast<char*>(ws) + gate_bytes;

    if (!preconcatenated) {
        ConcatParams cp;
        cp.x = input; cp.h = hidden; cp.out = ws;
        cp.x_m = x_m; cp.x_n = x_n; cp.h_m = h_m; cp.h_n = h_n;
        cp.rows = (uint32_t)rows; cp.nx = (uint32_t)nx; cp.nh = (uint32_t)nh;
        e = type == real32F ? launch_lstm_elementwise<float>(&cp, nullptr, stream)
            : type == real16F ? launch_lstm_elementwise<__half>(&cp, nullptr, stream)
                              : launch_lstm_elementwise<__nv_bfloat16>(&cp, nullptr, stream);
        if (e != cudaSuccess) return e;
    }

    // fused = gateInput . fusedWeight + fusedBias, rounded to the element type (what matmul(bias:) returns)
    size_t g_shape[2] = {(size_t)rows, (size_t)(nx + nh)};
    size_t g_strides[2] = {preconcatenated ? (size_t)x_m : (size_t)(nx + nh), preconcatenated ? (size_t)x_n : (size_t)1};
    size_t f_shape[2] = {(size_t)rows, (size_t)(4 * nh)}, f_strides[2] = {(size_t)(4 * nh), 1};
    srtTensorDescriptor gd, fd;
    memset(&gd, 0, sizeof gd);
    gd.type = type; gd.rank = 2; gd.order = srtOrderRow; gd.count = g_shape[0] * g_shape[1]; gd.spanCount = gd.count;
    gd.shape = g_shape; gd.strides = g_strides; gd.logicalStrides = g_strides;
    fd = gd;
    fd.strides = f_strides; fd.logicalStrides = f_strides;
    fd.count = f_shape[0] * f_shape[1]; fd.spanCount = fd.count;
    fd.shape = f_shape; fd.strides = f_strides; fd.logicalStrides = f_strides;
    e = srtMatmulBiasActivation(gate_in, &gd, false, fusedWeight, weightDesc, false, fusedBias, biasDesc, srtActivationIdentity,
                                fused, &fd, stream);
    if (e != cudaSuccess) return e;

    LstmGateParams gp;
    gp.fused = fused; gp.cell = cell; gp.new_cell = newCell; gp.new_hidden = newHidden;
    gp.c_m = c_m; gp.c_n = c_n; gp.nc_m = nc_m; gp.nc_n = nc_n; gp.nh_m = nh_m; gp.nh_n = nh_n;
    gp.rows = (uint32_t)rows; gp.hidden = (uint32_t)nh;
    return type == real32F ? launch_lstm_elementwise<float>(nullptr, &gp, stream)
           : type == real16F ? launch_lstm_elementwise<__half>(nullptr, &gp, stream)
                             : launch_lstm_elementwise<__nv_bfloat16>(nullptr, &gp, stream);
}

// ------------------------------------------------------------------ srtLstmCellFused
cudaError_t srtLstmInterleaveGates(const void* in, const srtTensorDescriptor* inDesc, void* out, const srtTensorDescriptor* outDesc,
                                   cudaStream_t stream)
{
    if (!in || !out || !inDesc || !outDesc || !inDesc->shape || !inDesc->strides || !outDesc->shape || !outDesc->strides)
        return fail(cudaErrorInvalidValue, "srtLstmInterleaveGates: null tensor or descriptor");
    if (inDesc->rank != outDesc->rank || (inDesc->rank != 1 && inDesc->rank != 2) || inDesc->type != outDesc->type)
        return fail(cudaErrorInvalidValue, "srtLstmInterleaveGates: in and out must be rank 1 or 2 tensors of one type and rank");
    const uint32_t q = inDesc->rank - 1;
    const uint64_t rows = inDesc->rank == 2 ? inDesc->shape[0] : 1, cols = inDesc->shape[q];
    if (cols % 4 || outDesc->shape[q] != cols || (inDesc->rank == 2 && outDesc->shape[0] != rows) || outDesc->strides[q] != 1)
        return fail(cudaErrorInvalidValue, "srtLstmInterleaveGates: 4 hiddenSize columns expected, out of the same shape with contiguous columns");
    if (elem_size(inDesc->type) == 0) return fail(cudaErrorNotSupported, "element type %d is not computed by this library", (int)inDesc->type);
    if (rows == 0 || cols == 0) return cudaSuccess;
    if (rows > 0xffffffffull || cols > 0xffffffffull) return fail(cudaErrorNotSupported, "srtLstmInterleaveGates: extents beyond 32 bits");
    DeviceScope scope(stream);
    if (scope.status != cudaSuccess) return scope.status;
    InterleaveParams ip;
    ip.in = in; ip.out = out;
    ip.in_m = inDesc->rank == 2 ? (long long)inDesc->strides[0] : 0; ip.in_n = (long long)inDesc->strides[q];
    ip.out_m = outDesc->rank == 2 ? (long long)outDesc->strides[0] : 0;
    ip.rows = (uint32_t)rows; ip.hidden = (uint32_t)(cols / 4);
    unsigned long long blocks = (rows * cols + 255) / 256;
    if (blocks > 148ull * 16) blocks = 148ull * 16;
    switch (inDesc->type) {
    case real32F: lstm_interleave_kernel<float><<<(unsigned)blocks, 256, 0, stream>>>(ip); break;
    case real16F: lstm_interleave_kernel<__half><<<(unsigned)blocks, 256, 0, stream>>>(ip); break;
    default: lstm_interleave_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, stream>>>(ip); break;
    }
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) g_launches.fetch_add(1, std::memory_order_relaxed);
    return e;
}

cudaError_t srtLstmCellFused(const void* input, const srtTensorDescriptor* inputDesc, const void* hidden,
                             const srtTensorDescriptor* hiddenDesc, const void* cell, const srtTensorDescriptor* cellDesc,
                             const void* interleavedWeight, const srtTensorDescriptor* weightDesc, const void* interleavedBias,
                             const srtTensorDescriptor* biasDesc, void* newCell, const srtTensorDescriptor* newCellDesc,
                             void* newHidden, const srtTensorDescriptor* newHiddenDesc, cudaStream_t stream)
{
    if (!input || !cell || !interleavedWeight || !newCell || !newHidden || !inputDesc)
        return fail(cudaErrorInvalidValue, "srtLstmCellFused: null tensor");
    const srtDataType type = inputDesc->type;
    if (type != real16F && type != real16BF)
        return fail(cudaErrorNotSupported, "srtLstmCellFused: 16-bit element types only; use srtLstmCell");
    uint64_t rows, nx, r2, nh, r3, c3, wk, wn, r4, c4, r5, c5;
    long long x_m, x_n, h_m = 0, h_n = 0, c_m, c_n, w_m, w_n, nc_m, nc_n, nh_m, nh_n;
    cudaError_t e;
    if ((e = view2(inputDesc, "input", type, rows, nx, x_m, x_n)) != cudaSuccess) return e;
    const bool preconcatenated = hidden == nullptr;
    if ((e = view2(cellDesc, "cell", type, r3, c3, c_m, c_n)) != cudaSuccess) return e;
    nh = c3;
    if (preconcatenated) {
        if (nx < nh) return fail(cudaErrorInvalidValue, "srtLstmCellFused: a gate input has at least hiddenSize columns");
        nx -= nh;
        r2 = rows;
    } else {
        uint64_t hcols;
        if ((e = view2(hiddenDesc, "hidden", type, r2, hcols, h_m, h_n)) != cudaSuccess) return e;
        if (hcols != nh) return fail(cudaErrorInvalidValue, "srtLstmCellFused: hidden and cell must have the same shape");
    }
    if ((e = view2(weightDesc, "interleavedWeight", type, wk, wn, w_m, w_n)) != cudaSuccess) return e;
    if ((e = view2(newCellDesc, "newCell", type, r4, c4, nc_m, nc_n)) != cudaSuccess) return e;
    if ((e = view2(newHiddenDesc, "newHidden", type, r5, c5, nh_m, nh_n)) != cudaSuccess) return e;
    if (r2 != rows || r3 != rows || r4 != rows || r5 != rows || c4 != nh || c5 != nh)
        return fail(cudaErrorInvalidValue, "srtLstmCellFused: state tensors must be [batch x hiddenSize]");
    if (wk != nx + nh || wn != 4 * nh)
        return fail(cudaErrorInvalidValue, "srtLstmCellFused: interleavedWeight must be [(inputSize + hiddenSize) x 4 hiddenSize]");
    if (interleavedBias && (!biasDesc || biasDesc->rank != 1 || biasDesc->shape[0] != 4 * nh || biasDesc->type != type))
        return fail(cudaErrorInvalidValue, "srtLstmCellFused: interleavedBias must be rank 1 with 4 hiddenSize elements");
    if (rows == 0 || nh == 0) return cudaSuccess;
    // the epilogue moves 8 hidden units (16 bytes) per access
    const bool state_ok = nh % 8 == 0 && c_n == 1 && nc_n == 1 && nh_n == 1 && aligned16(cell, c_m, 2) && aligned16(newCell, nc_m, 2) &&
                          aligned16(newHidden, nh_m, 2);
    if (!state_ok || rows > 0x7fffffffull || nx + nh > 0x7fffffffull)
        return fail(cudaErrorNotSupported, "srtLstmCellFused: hiddenSize must be a multiple of 8 and the state tensors row-contiguous and "
                                           "16-byte aligned; use srtLstmCell");
    DeviceScope scope(stream);
    if (scope.status != cudaSuccess) return scope.status;

    // the gate input: the caller's, or the concatenation staged in the workspace
    const void* gate_in = input;
    long long g_m = x_m, g_n = x_n;
    if (!preconcatenated) {
        void* ws = nullptr;
        if ((e = workspace_for(scope.device, stream, (size_t)rows * (nx + nh) * 2, &ws, 1)) != cudaSuccess) return e;
        ConcatParams cp;
        cp.x = input; cp.h = hidden; cp.out = ws;
        cp.x_m = x_m; cp.x_n = x_n; cp.h_m = h_m; cp.h_n = h_n;
        cp.rows = (uint32_t)rows; cp.nx = (uint32_t)nx; cp.nh = (uint32_t)nh;
        e = type == real16F ? launch_lstm_elementwise<__half>(&cp, nullptr, stream) : launch_lstm_elementwise<__nv_bfloat16>(&cp, nullptr, stream);
        if (e != cudaSuccess) return e;
        gate_in = ws; g_m = (long long)(nx + nh); g_n = 1;
    }
    // the product [batch x (inputSize + hiddenSize)] . [.. x 4 hiddenSize] as the planner sees it; its "result" is never stored
    Problem P;
    memset(&P, 0, sizeof P);
    P.type = type; P.elem = 2;
    P.batch = 1; P.M = rows; P.N = 4 * nh; P.K = nx + nh;
    P.a = static_cast<const char*>(gate_in); P.a_m = g_m; P.a_k = g_n;
    P.b = static_cast<const char*>(interleavedWeight); P.b_k = w_m; P.b_n = w_n;
    P.out = static_cast<char*>(newCell);               // an aligned stand-in: the LSTM epilogue writes no product
    P.o_m = (long long)(4 * nh); P.o_n = 1;
    P.bias = static_cast<const char*>(interleavedBias); P.bias_stride = interleavedBias ? (long long)biasDesc->strides[0] : 0;
    P.act = kActIdentity;
    Plan plan;
    if ((e = plan_for(P, plan)) != cudaSuccess) return e;
    if ((plan.pub.kernel != srtMatmulKernelTcgen05 && plan.pub.kernel != srtMatmulKernelTcgen05Pair) || plan.splits > 1 || plan.swapped)
        return fail(cudaErrorNotSupported, "srtLstmCellFused: this product does not run on a 16-bit tensor-core kernel in one pass; use srtLstmCell");
    std::unique_ptr<Prepared> pr(new Prepared());
    if ((e = prepare_tc(plan, *pr)) != cudaSuccess) return e;
    GemmParams& gp = pr->gp;
    gp.epilogue = kEpilogueLstm;
    gp.out = nullptr; gp.out_tma = 0;
    gp.lstm_cell = cell; gp.lstm_new_cell = newCell; gp.lstm_new_hidden = newHidden;
    gp.lstm_c_m = c_m; gp.lstm_nc_m = nc_m; gp.lstm_nh_m = nh_m;
    return launch_prepared(*pr, stream);
}

// ------------------------------------------------------------------ srtRnnCell
cudaError_t srtRnnCell(const void* input, const srtTensorDescriptor* inputDesc, const void* hidden,
                       const srtTensorDescriptor* hiddenDesc, const void* weight, const srtTensorDescriptor* weightDesc,
                       const void* bias, const srtTensorDescriptor* biasDesc, void* newHidden,
                       const srtTensorDescriptor* newHiddenDesc, cudaStream_t stream)
{
    if (!input || !hidden || !weight || !newHidden || !inputDesc)
        return fail(cudaErrorInvalidValue, "srtRnnCell: null tensor");
    const srtDataType type = inputDesc->type;
    if (type != real32F && type != real16F && type != real16BF)
        return fail(cudaErrorNotSupported, "srtRnnCell: element type %d is outside this library", (int)type);
    uint64_t rows, nx, r2, nh, wk, wn, r3, c3;
    long long x_m, x_n, h_m, h_n, w_m, w_n, o_m, o_n;
    cudaError_t e;
    if ((e = view2(inputDesc, "input", type, rows, nx, x_m, x_n)) != cudaSuccess) return e;
    if ((e = view2(hiddenDesc, "hidden", type, r2, nh, h_m, h_n)) != cudaSuccess) return e;
    if ((e = view2(weightDesc, "weight", type, wk, wn, w_m, w_n)) != cudaSuccess) return e;
    if ((e = view2(newHiddenDesc, "newHidden", type, r3, c3, o_m, o_n)) != cudaSuccess) return e;
    if (r2 != rows || r3 != rows || c3 != nh || wk != nx + nh || wn != nh)
        return fail(cudaErrorInvalidValue, "srtRnnCell: weight must be [(inputSize + hiddenSize) x hiddenSize], states [batch x hiddenSize]");
    // the reference keeps the bias as a [1 x hiddenSize] matrix (Recurrent.swift:139); a vector is accepted too
    srtTensorDescriptor bias1;
    size_t b_shape[1], b_strides[1];
    if (bias) {
        if (!biasDesc || biasDesc->type != type || !biasDesc->shape || !biasDesc->strides)
            return fail(cudaErrorInvalidValue, "srtRnnCell: bias without a matching descriptor");
        const bool vec = biasDesc->rank == 1 && biasDesc->shape[0] == nh;
        const bool row = biasDesc->rank == 2 && biasDesc->shape[0] == 1 && biasDesc->shape[1] == nh;
        if (!vec && !row) return fail(cudaErrorInvalidValue, "srtRnnCell: bias must be [hiddenSize] or [1 x hiddenSize]");
        bias1 = *biasDesc;
        bias1.rank = 1;
        b_shape[0] = (size_t)nh;
        b_strides[0] = vec ? biasDesc->strides[0] : biasDesc->strides[1];
        bias1.shape = b_shape; bias1.strides = b_strides; bias1.logicalStrides = b_strides;
        bias1.count = (size_t)nh; bias1.spanCount = 1 + (size_t)(nh - 1) * b_strides[0];
    }
    if (rows == 0 || nh == 0) return cudaSuccess;
    if (rows > 0xffffffffull || nx + nh > 0xffffffffull) return fail(cudaErrorNotSupported, "srtRnnCell: extents beyond 32 bits");
    const size_t elem = type == real32F ? 4 : 2;
    DeviceScope scope(stream);
    if (scope.status != cudaSuccess) return scope.status;
    const int dev = scope.device;
    void* gate_in = nullptr;
    if ((e = workspace_for(dev, stream, (size_t)rows * (nx + nh) * elem, &gate_in, 1)) != cudaSuccess) return e;
    ConcatParams cp;
    cp.x = input; cp.h = hidden; cp.out = gate_in;
    cp.x_m = x_m; cp.x_n = x_n; cp.h_m = h_m; cp.h_n = h_n;
    cp.rows = (uint32_t)rows; cp.nx = (uint32_t)nx; cp.nh = (uint32_t)nh;
    e = type == real32F ? launch_lstm_elementwise<float>(&cp, nullptr, stream)
        : type == real16F ? launch_lstm_elementwise<__half>(&cp, nullptr, stream)
                          : launch_lstm_elementwise<__nv_bfloat16>(&cp, nullptr, stream);
    if (e != cudaSuccess) return e;
    size_t g_shape[2] = {(size_t)rows, (size_t)(nx + nh)}, g_strides[2] = {(size_t)(nx + nh), 1};
    srtTensorDescriptor gd;
    memset(&gd, 0, sizeof gd);
    gd.type = type; gd.rank = 2; gd.order = srtOrderRow; gd.count = g_shape[0] * g_shape[1]; gd.spanCount = gd.count;
    gd.shape = g_shape; gd.strides = g_strides; gd.logicalStrides = g_strides;
    // newState = tanh(matmul(concatenate(input, state), weight) + bias): the fused epilogue does the rest
    return srtMatmulBiasActivation(gate_in, &gd, false, weight, weightDesc, false, bias, bias ? &bias1 : nullptr, srtActivationTanh,
                                   newHidden, newHiddenDesc, stream);
}

// ------------------------------------------------------------------ srtGruCell
cudaError_t srtGruCell(const void* input, const srtTensorDescriptor* inputDesc, const void* hidden,
                       const srtTensorDescriptor* hiddenDesc, const void* gateWeight, const srtTensorDescriptor* gateWeightDesc,
                       const void* gateBias, const srtTensorDescriptor* gateBiasDesc, const void* outputWeight,
                       const srtTensorDescriptor* outputWeightDesc, const void* outputBias,
                       const srtTensorDescriptor* outputBiasDesc, void* newHidden, const srtTensorDescriptor* newHiddenDesc,
                       cudaStream_t stream)
{
    if (!input || !hidden || !gateWeight || !outputWeight || !newHidden || !inputDesc)
        return fail(cudaErrorInvalidValue, "srtGruCell: null tensor");
    const srtDataType type = inputDesc->type;
    if (type != real32F && type != real16F && type != real16BF)
        return fail(cudaErrorNotSupported, "srtGruCell: element type %d is outside this library", (int)type);
    uint64_t rows, nx, r2, nh, gk, gn, ok, on, r3, c3;
    long long x_m, x_n, h_m, h_n, g_m, g_n, o_m, o_n, nh_m, nh_n;
    cudaError_t e;
    if ((e = view2(inputDesc, "input", type, rows, nx, x_m, x_n)) != cudaSuccess) return e;
    if ((e = view2(hiddenDesc, "hidden", type, r2, nh, h_m, h_n)) != cudaSuccess) return e;
    if ((e = view2(gateWeightDesc, "gateWeight", type, gk, gn, g_m, g_n)) != cudaSuccess) return e;
    if ((e = view2(outputWeightDesc, "outputWeight", type, ok, on, o_m, o_n)) != cudaSuccess) return e;
    if ((e = view2(newHiddenDesc, "newHidden", type, r3, c3, nh_m, nh_n)) != cudaSuccess) return e;
    if (r2 != rows || r3 != rows || c3 != nh || gk != nx + nh || gn != 2 * nh || ok != nx + nh || on != nh)
        return fail(cudaErrorInvalidValue,
                    "srtGruCell: gateWeight must be [(inputSize + hiddenSize) x 2 hiddenSize], outputWeight [(inputSize + hiddenSize) x "
                    "hiddenSize], states [batch x hiddenSize]");
    if (gateBias && (!gateBiasDesc || gateBiasDesc->rank != 1 || gateBiasDesc->shape[0] != 2 * nh || gateBiasDesc->type != type))
        return fail(cudaErrorInvalidValue, "srtGruCell: gateBias must be rank 1 with 2 hiddenSize elements");
    if (outputBias && (!outputBiasDesc || outputBiasDesc->rank != 1 || outputBiasDesc->shape[0] != nh || outputBiasDesc->type != type))
        return fail(cudaErrorInvalidValue, "srtGruCell: outputBias must be rank 1 with hiddenSize elements");
    if (rows == 0 || nh == 0) return cudaSuccess;
    if (rows > 0xffffffffull || nx + nh > 0xffffffffull || 2 * nh > 0xffffffffull)
        return fail(cudaErrorNotSupported, "srtGruCell: extents beyond 32 bits");
    DeviceScope scope(stream);
    if (scope.status != cudaSuccess) return scope.status;

    const size_t elem = type == real32F ? 4 : 2;
    auto pad = [](size_t n) { return (n + 255) & ~(size_t)255; };
    const size_t cat_bytes = pad((size_t)rows * (nx + nh) * elem), gates_bytes = pad((size_t)rows * 2 * nh * elem);
    const size_t out_bytes = (size_t)rows * nh * elem;
    void* ws = nullptr;
    if ((e = workspace_for(scope.device, stream, cat_bytes + gates_bytes + out_bytes, &ws, 1)) != cudaSuccess) return e;
    void* cat = ws;
    void* gates = static_cast<char*>(ws) + cat_bytes;
    void* outv = static_cast<char*>(gates) + gates_bytes;

    ConcatParams cp;
    cp.x = input; cp.h = hidden; cp.out = cat;
    cp.x_m = x_m; cp.x_n = x_n; cp.h_m = h_m; cp.h_n = h_n;
    cp.rows = (uint32_t)rows; cp.nx = (uint32_t)nx; cp.nh = (uint32_t)nh;
    e = type == real32F ? launch_lstm_elementwise<float>(&cp, nullptr, stream)
        : type == real16F ? launch_lstm_elementwise<__half>(&cp, nullptr, stream)
                          : launch_lstm_elementwise<__nv_bfloat16>(&cp, nullptr, stream);
    if (e != cudaSuccess) return e;

    size_t c_shape[2] = {(size_t)rows, (size_t)(nx + nh)}, c_strides[2] = {(size_t)(nx + nh), 1};
    size_t g_shape[2] = {(size_t)rows, (size_t)(2 * nh)}, g_strides[2] = {(size_t)(2 * nh), 1};
    size_t o_shape[2] = {(size_t)rows, (size_t)nh}, o_strides[2] = {(size_t)nh, 1};
    auto dense2 = [&](size_t* shape, size_t* strides) {
        srtTensorDescriptor d;
        memset(&d, 0, sizeof d);
        d.type = type; d.rank = 2; d.order = srtOrderRow; d.count = shape[0] * shape[1]; d.spanCount = d.count;
        d.shape = shape; d.strides = strides; d.logicalStrides = strides;
        return d;
    };
    const srtTensorDescriptor cd = dense2(c_shape, c_strides), gd = dense2(g_shape, g_strides), od = dense2(o_shape, o_strides);
    // reset | update = sigmoid([x | h] . gateWeight + gateBias)
    e = srtMatmulBiasActivation(cat, &cd, false, gateWeight, gateWeightDesc, false, gateBias, gateBiasDesc, srtActivationSigmoid,
                                gates, &gd, stream);
    if (e != cudaSuccess) return e;
    GruParams gp;
    gp.gate_in = cat; gp.gates = gates; gp.output = outv; gp.hidden = hidden; gp.new_hidden = newHidden;
    gp.h_m = h_m; gp.h_n = h_n; gp.nh_m = nh_m; gp.nh_n = nh_n;
    gp.rows = (uint32_t)rows; gp.nx = (uint32_t)nx; gp.nh = (uint32_t)nh;
    unsigned long long blocks64 = ((unsigned long long)rows * nh + 255) / 256;
    const unsigned blocks = (unsigned)(blocks64 < 148ull * 16 ? blocks64 : 148ull * 16);
    switch (type) {
    case real32F: gru_reset_kernel<float><<<blocks, 256, 0, stream>>>(gp); break;
    case real16F: gru_reset_kernel<__half><<<blocks, 256, 0, stream>>>(gp); break;
    default: gru_reset_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(gp); break;
    }
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    g_launches.fetch_add(1, std::memory_order_relaxed);
    // output = tanh([x | reset * h] . outputWeight + outputBias)
    e = srtMatmulBiasActivation(cat, &cd, false, outputWeight, outputWeightDesc, false, outputBias, outputBiasDesc, srtActivationTanh,
                                outv, &od, stream);
    if (e != cudaSuccess) return e;
    switch (type) {
    case real32F: gru_state_kernel<float><<<blocks, 256, 0, stream>>>(gp); break;
    case real16F: gru_state_kernel<__half><<<blocks, 256, 0, stream>>>(gp); break;
    default: gru_state_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(gp); break;
    }
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return cudaSuccess;
}

// ------------------------------------------------------------------ sharding over GPUs
cudaError_t srtShardRange(size_t total, int32_t world, int32_t rank, size_t align, size_t* start, size_t* stop)
{
    if (!start || !stop) return fail(cudaErrorInvalidValue, "srtShardRange: null result");
    if (world < 1 || rank < 0 || rank >= world) return fail(cudaErrorInvalidValue, "srtShardRange: rank %d outside a world of %d", rank, world);
    if (align == 0) align = 1;
    const size_t units = (total + align - 1) / align;
    const size_t base = units / (size_t)world, extra = units % (size_t)world;
    const size_t r = (size_t)rank;
    const size_t start_u = r * base + (r < extra ? r : extra);
    const size_t stop_u = start_u + base + (r < extra ? 1 : 0);
    *start = start_u * align < total ? start_u * align : total;
    *stop = stop_u * align < total ? stop_u * align : total;
    return cudaSuccess;
}

namespace {

// A descriptor with its own copies of the shape / stride arrays, narrowed along one dimension.
struct SlicedTensor {
    srtTensorDescriptor desc;
    size_t shape[3], strides[3];
    const char* ptr = nullptr;
    void init(const void* base, const srtTensorDescriptor* d)
    {
        desc = *d;
        for (uint32_t i = 0; i < d->rank && i < 3; ++i) { shape[i] = d->shape[i]; strides[i] = d->strides[i]; }
        desc.shape = shape; desc.strides = strides; desc.logicalStrides = strides;
        ptr = static_cast<const char*>(base);
    }
    void narrow(uint32_t dim, size_t lo, size_t hi, size_t elem)
    {
        ptr += lo * strides[dim] * elem;
        shape[dim] = hi - lo;
        size_t count = 1, span = 1;
        for (uint32_t i = 0; i < desc.rank; ++i) { count *= shape[i]; span += (shape[i] ? shape[i] - 1 : 0) * strides[i]; }
        desc.count = count;
        desc.spanCount = count ? span : 0;
    }
};

}  // namespace

cudaError_t srtMatmulSharded(srtShardAxis axis, int32_t world, int32_t rank, const void* a, const srtTensorDescriptor* aDesc,
                             bool transA, const void* b, const srtTensorDescriptor* bDesc, bool transB, const void* bias,
                             const srtTensorDescriptor* biasDesc, srtActivationType activation, void* out,
                             const srtTensorDescriptor* oDesc, int32_t peerCount, void* const* peerOut, void* multicastOut,
                             cudaStream_t stream)
{
    if (!aDesc || !bDesc || !oDesc || !aDesc->shape || !bDesc->shape || !oDesc->shape || !aDesc->strides || !bDesc->strides ||
        !oDesc->strides)
        return fail(cudaErrorInvalidValue, "srtMatmulSharded: null descriptor");
    if (aDesc->rank < 2 || aDesc->rank > 3 || bDesc->rank < 2 || bDesc->rank > 3 || oDesc->rank < 2 || oDesc->rank > 3)
        return fail(cudaErrorNotSupported, "srtMatmulSharded: tensors of rank 2 or 3 expected");
    if (peerCount < 0 || peerCount > (int32_t)kMaxPeers || (peerCount > 0 && !peerOut))
        return fail(cudaErrorInvalidValue, "srtMatmulSharded: peerCount %d outside 0..%u, or null peerOut", peerCount, kMaxPeers);
    const size_t elem = elem_size(oDesc->type);
    if (elem == 0) return fail(cudaErrorNotSupported, "element type %d is not computed by this library", (int)oDesc->type);
    SlicedTensor sa, sb, so, sbias;
    sa.init(a, aDesc); sb.init(b, bDesc); so.init(out, oDesc);
    const uint32_t aq = aDesc->rank - 2, bq = bDesc->rank - 2, oq = oDesc->rank - 2;
    size_t total = 0, align = 1;
    switch (axis) {
    case srtShardBatch:
        if (oDesc->rank != 3) return fail(cudaErrorInvalidValue, "srtMatmulSharded: batch sharding needs a rank-3 result");
        total = oDesc->shape[0];
        break;
    case srtShardM: total = oDesc->shape[oq]; break;
    case srtShardN: total = oDesc->shape[oq + 1]; align = 16 / elem; break;       // column blocks stay 16-byte aligned
    default: return fail(cudaErrorInvalidValue, "srtMatmulSharded: unknown axis %d", (int)axis);
    }
    size_t lo = 0, hi = 0;
    cudaError_t e = srtShardRange(total, world, rank, align, &lo, &hi);
    if (e != cudaSuccess) return e;
    if (hi <= lo) return cudaSuccess;                                              // more ranks than blocks: nothing for this one
    const void* bias_ptr = bias;
    const srtTensorDescriptor* bias_desc = biasDesc;
    uint32_t odim = 0;
    if (axis == srtShardBatch) {
        if (aDesc->rank == 3 && aDesc->shape[0] != 1) sa.narrow(0, lo, hi, elem);
        if (bDesc->rank == 3 && bDesc->shape[0] != 1) sb.narrow(0, lo, hi, elem);
        odim = 0;
    } else if (axis == srtShardM) {
        sa.narrow(aq + (transA ? 1 : 0), lo, hi, elem);
        odim = oq;
    } else {
        sb.narrow(bq + (transB ? 0 : 1), lo, hi, elem);
        odim = oq + 1;
        if (bias) {
            if (!biasDesc || biasDesc->rank != 1 || !biasDesc->shape || !biasDesc->strides)
                return fail(cudaErrorInvalidValue, "srtMatmulSharded: bias must be rank 1");
            sbias.init(bias, biasDesc);
            sbias.narrow(0, lo, hi, elem);
            bias_ptr = sbias.ptr;
            bias_desc = &sbias.desc;
        }
    }
    const size_t out_offset = lo * so.strides[odim] * elem;
    so.narrow(odim, lo, hi, elem);
    void* peers[kMaxPeers];
    for (int32_t i = 0; i < peerCount; ++i) {
        if (!peerOut[i]) return fail(cudaErrorInvalidValue, "srtMatmulSharded: peerOut[%d] is null", i);
        peers[i] = static_cast<char*>(peerOut[i]) + out_offset;
    }
    void* mc = multicastOut ? static_cast<char*>(multicastOut) + out_offset : nullptr;
    void* out_view = const_cast<char*>(so.ptr);
    if (mc) {
        e = srtMatmulAllGatherMulticast(sa.ptr, &sa.desc, transA, sb.ptr, &sb.desc, transB, bias_ptr, bias_desc, activation, out_view,
                                        &so.desc, mc, stream);
        if (e != cudaErrorNotSupported || peerCount == 0) return e;             // not eligible: peer by peer instead
    }
    if (peerCount > 0)
        return srtMatmulAllGather(sa.ptr, &sa.desc, transA, sb.ptr, &sb.desc, transB, bias_ptr, bias_desc, activation, out_view,
                                  &so.desc, peerCount, peers, stream);
    return srtMatmulBiasActivation(sa.ptr, &sa.desc, transA, sb.ptr, &sb.desc, transB, bias_ptr, bias_desc, activation, out_view,
                                   &so.desc, stream);
}

cudaError_t srtMatmulShardedDevices(srtShardAxis axis, int32_t nDevices, const cudaStream_t* streams, const void* const* a,
                                    const srtTensorDescriptor* aDesc, bool transA, const void* const* b,
                                    const srtTensorDescriptor* bDesc, bool transB, const void* const* bias,
                                    const srtTensorDescriptor* biasDesc, srtActivationType activation, void* const* out,
                                    const srtTensorDescriptor* oDesc, bool gather, void* multicastOut)
{
    if (nDevices < 1 || nDevices > (int32_t)kMaxPeers + 1 || !streams || !a || !b || !out)
        return fail(cudaErrorInvalidValue, "srtMatmulShardedDevices: 1..%u devices with their streams and buffers expected", kMaxPeers + 1);
    int devices[kMaxPeers + 1];
    for (int32_t i = 0; i < nDevices; ++i) {
        DeviceScope scope(streams[i]);
        if (scope.status != cudaSuccess) return scope.status;
        devices[i] = scope.device;
    }
    if (gather && nDevices > 1) {
        // every device stores into every other device's result buffer: one process, so plain peer access
        for (int32_t i = 0; i < nDevices; ++i) {
            DeviceScope scope(streams[i]);
            for (int32_t j = 0; j < nDevices; ++j) {
                if (devices[j] == devices[i]) continue;
                int can = 0;
                cudaError_t e = cudaDeviceCanAccessPeer(&can, devices[i], devices[j]);
                if (e != cudaSuccess) return e;
                if (!can) return fail(cudaErrorNotSupported, "srtMatmulShardedDevices: device %d cannot address device %d", devices[i], devices[j]);
                e = cudaDeviceEnablePeerAccess(devices[j], 0);
                if (e == cudaErrorPeerAccessAlreadyEnabled) (void)cudaGetLastError();
                else if (e != cudaSuccess) return fail(e, "cudaDeviceEnablePeerAccess(%d -> %d) failed: %s", devices[i], devices[j], cudaGetErrorString(e));
            }
        }
    }
    for (int32_t i = 0; i < nDevices; ++i) {
        void* peers[kMaxPeers];
        int32_t count = 0;
        if (gather)
            for (int32_t j = 0; j < nDevices; ++j)
                if (j != i) peers[count++] = out[j];
        cudaError_t e = srtMatmulSharded(axis, nDevices, i, a[i], aDesc, transA, b[i], bDesc, transB, bias ? bias[i] : nullptr, biasDesc,
                                         activation, out[i], oDesc, count, peers, gather ? multicastOut : nullptr, streams[i]);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

// ------------------------------------------------------------------ NVLink multicast buffers (one process, several devices)
cudaError_t srtMulticastAlloc(int32_t nDevices, const int32_t* devices, size_t bytes, void** localPtrs, void** multicastPtr,
                              srtMulticastBuffer* handle)
{
    if (nDevices < 2 || nDevices > (int32_t)kMaxPeers + 1 || !devices || !localPtrs || !multicastPtr || !handle || bytes == 0)
        return fail(cudaErrorInvalidValue, "srtMulticastAlloc: 2..%u devices, a size and result pointers expected", kMaxPeers + 1);
    const DriverApi& d = driver_api();
    if (!d.ok) return fail(cudaErrorNotSupported, "srtMulticastAlloc: the driver does not export the multicast entry points");
    int cur = 0;
    cudaError_t ce = cudaGetDevice(&cur);
    if (ce != cudaSuccess) return ce;
    for (int32_t i = 0; i < nDevices; ++i) {
        if ((ce = cudaSetDevice(devices[i])) != cudaSuccess || (ce = cudaFree(nullptr)) != cudaSuccess) {      // primary context up
            cudaSetDevice(cur);
            return fail(ce, "srtMulticastAlloc: device %d: %s", devices[i], cudaGetErrorString(ce));
        }
        int supported = 0;
        if (d.DeviceGetAttribute(&supported, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, devices[i]) != CUDA_SUCCESS || !supported) {
            cudaSetDevice(cur);
            return fail(cudaErrorNotSupported, "srtMulticastAlloc: device %d has no NVLink multicast", devices[i]);
        }
    }
    MulticastBuffer* b = new MulticastBuffer();
    b->n = nDevices;
    for (int32_t i = 0; i < nDevices; ++i) b->devices[i] = devices[i];
    CUmulticastObjectProp prop;
    memset(&prop, 0, sizeof prop);
    prop.numDevices = (unsigned)nDevices;
    prop.size = bytes;
    size_t gran = 0;
    CUresult r = d.MulticastGetGranularity(&gran, &prop, CU_MULTICAST_GRANULARITY_RECOMMENDED);
    auto bail = [&](const char* what, CUresult code) {
        multicast_destroy(b);
        cudaSetDevice(cur);
        return fail(code == CUDA_ERROR_NOT_SUPPORTED || code == CUDA_ERROR_NOT_PERMITTED ? cudaErrorNotSupported : cudaErrorUnknown,
                    "srtMulticastAlloc: %s failed with driver code %d", what, (int)code);
    };
    if (r != CUDA_SUCCESS || gran == 0) return bail("cuMulticastGetGranularity", r);
    b->size = (bytes + gran - 1) / gran * gran;
    prop.size = b->size;
    if ((r = d.MulticastCreate(&b->mc, &prop)) != CUDA_SUCCESS) { b->mc = 0; return bail("cuMulticastCreate", r); }
    for (int32_t i = 0; i < nDevices; ++i)
        if ((r = d.MulticastAddDevice(b->mc, devices[i])) != CUDA_SUCCESS) return bail("cuMulticastAddDevice", r);
    CUmemAccessDesc access[kMaxPeers + 1];
    for (int32_t i = 0; i < nDevices; ++i) {
        access[i].location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        access[i].location.id = devices[i];
        access[i].flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    }
    for (int32_t i = 0; i < nDevices; ++i) {
        CUmemAllocationProp ap;
        memset(&ap, 0, sizeof ap);
        ap.type = CU_MEM_ALLOCATION_TYPE_PINNED;
        ap.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        ap.location.id = devices[i];
        if ((r = d.MemCreate(&b->mem[i], b->size, &ap, 0)) != CUDA_SUCCESS) { b->mem[i] = 0; return bail("cuMemCreate", r); }
        if ((r = d.MulticastBindMem(b->mc, 0, b->mem[i], 0, b->size, 0)) != CUDA_SUCCESS) return bail("cuMulticastBindMem", r);
        b->bound[i] = true;
        if ((r = d.MemAddressReserve(&b->va[i], b->size, gran, 0, 0)) != CUDA_SUCCESS) { b->va[i] = 0; return bail("cuMemAddressReserve", r); }
        if ((r = d.MemMap(b->va[i], b->size, 0, b->mem[i], 0)) != CUDA_SUCCESS) return bail("cuMemMap", r);
        if ((r = d.MemSetAccess(b->va[i], b->size, access, (size_t)nDevices)) != CUDA_SUCCESS) return bail("cuMemSetAccess", r);
    }
    if ((r = d.MemAddressReserve(&b->mc_va, b->size, gran, 0, 0)) != CUDA_SUCCESS) { b->mc_va = 0; return bail("cuMemAddressReserve (multicast)", r); }
    if ((r = d.MemMap(b->mc_va, b->size, 0, b->mc, 0)) != CUDA_SUCCESS) return bail("cuMemMap (multicast)", r);
    if ((r = d.MemSetAccess(b->mc_va, b->size, access, (size_t)nDevices)) != CUDA_SUCCESS) return bail("cuMemSetAccess (multicast)", r);
    for (int32_t i = 0; i < nDevices; ++i) localPtrs[i] = reinterpret_cast<void*>(b->va[i]);
    *multicastPtr = reinterpret_cast<void*>(b->mc_va);
    *handle = b;
    cudaSetDevice(cur);
    return cudaSuccess;
}

cudaError_t srtMulticastFree(srtMulticastBuffer handle)
{
    if (!handle) return cudaSuccess;
    int cur = 0;
    cudaGetDevice(&cur);
    multicast_destroy(static_cast<MulticastBuffer*>(handle));
    cudaSetDevice(cur);
    return cudaSuccess;
}

cudaError_t srtMatmulSetWaitLimit(uint64_t nanoseconds)
{
    g_wait_limit_ns.store(nanoseconds ? nanoseconds : (uint64_t)srt::kDefaultWaitLimitNs, std::memory_order_relaxed);
    return cudaSuccess;
}

// ------------------------------------------------------------------ srtMatmulNoAlloc
cudaError_t srtMatmulNoAlloc(const void* a, const srtTensorDescriptor* aDesc, bool transA, const void* b,
                             const srtTensorDescriptor* bDesc, bool transB, void* out, const srtTensorDescriptor* oDesc,
                             cudaStream_t stream)
{
    // The same planning, call cache and launches as srtMatmul.  A split-K plan binds its partial sums
    // to the static array: the first pass writes every element of every slice before the second pass
    // reads it, so nothing in the array has to start at zero and what an earlier call left is harmless.
    return run_matmul(a, aDesc, transA, b, bDesc, transB, nullptr, nullptr, srtActivationIdentity, out, oDesc, stream, true);
}

// ------------------------------------------------------------------ srtMatmulAllGather
// One rank's part of "every GPU computes a block of C, every GPU ends up with all of C".
// `out` is this rank's block as a view into its own full-size buffer; peerOut[i] is the first
// element of the SAME view in the buffer of another GPU, mapped into this process (see
// srtPeerMemOpen).  When the plan is the CTA-pair kernel with bulk tensor stores, the epilogue
// stores each finished tile to all buffers (one kernel: the transfers overlap the product tile by
// tile).  Any other plan runs the ordinary product and then copies the block to each peer on the
// same stream.  Nothing waits for another GPU: the peers' copies are complete when this stream
// has drained, and the caller synchronises the ranks (a host barrier) before anyone reads.
struct GatherKey {
    CallKey call;
    void* peers[kMaxPeers];
    void* multicast;
    int32_t count;
    int32_t pad;
};
struct GatherEntry {
    bool valid = false;
    bool fused = false;
    GatherKey key;
    Prepared pr;
    PeerMaps maps;
};
constexpr int kGatherCacheSize = 8;
static thread_local std::unique_ptr<GatherEntry[]> t_gather;

static cudaError_t copy_view_to_peers(const Problem& P, const srtTensorDescriptor* oDesc, const void* out, int32_t count,
                               void* const* peers, cudaStream_t stream)
{
    View3 v;
    cudaError_t e = view3(oDesc, "out", v);
    if (e != cudaSuccess) return e;
    size_t width, height, pitch;
    if (v.s_n == 1 || v.N == 1) { width = v.N * P.elem; height = v.M; pitch = (size_t)v.s_m * P.elem; }
    else if (v.s_m == 1 || v.M == 1) { width = v.M * P.elem; height = v.N; pitch = (size_t)v.s_n * P.elem; }
    else return fail(cudaErrorNotSupported, "srtMatmulAllGather: the output view has no contiguous dimension");
    if (height <= 1) pitch = width;
    if (pitch < width) return fail(cudaErrorNotSupported, "srtMatmulAllGather: overlapping output rows");
    for (int32_t i = 0; i < count; ++i)
        for (uint64_t bt = 0; bt < v.batch; ++bt) {
            const size_t off = (size_t)bt * (size_t)v.s_b * P.elem;
            e = cudaMemcpy2DAsync(static_cast<char*>(peers[i]) + off, pitch, static_cast<const char*>(out) + off, pitch, width,
                                  height, cudaMemcpyDefault, stream);
            if (e != cudaSuccess) return fail(e, "srtMatmulAllGather: copy to peer %d failed: %s", i, cudaGetErrorString(e));
        }
    return cudaSuccess;
}

static cudaError_t gather_impl(const void* a, const srtTensorDescriptor* aDesc, bool transA, const void* b,
                               const srtTensorDescriptor* bDesc, bool transB, const void* bias,
                               const srtTensorDescriptor* biasDesc, srtActivationType activation, void* out,
                               const srtTensorDescriptor* oDesc, int32_t peerCount, void* const* peerOut, void* multicastOut,
                               cudaStream_t stream)
{
    if (peerCount < 0 || peerCount > (int32_t)kMaxPeers)
        return fail(cudaErrorInvalidValue, "srtMatmulAllGather: peerCount %d outside 0..%u", peerCount, kMaxPeers);
    if (peerCount > 0 && !peerOut) return fail(cudaErrorInvalidValue, "srtMatmulAllGather: null peerOut");
    if (peerCount == 0 && !multicastOut)
        return srtMatmulBiasActivation(a, aDesc, transA, b, bDesc, transB, bias, biasDesc, activation, out, oDesc, stream);
    GatherKey key;
    memset(&key, 0, sizeof key);
    Problem& P = key.call.P;
    cudaError_t e = parse(a, aDesc, transA, b, bDesc, transB, bias, biasDesc, (int)activation, out, oDesc, P);
    if (e != cudaSuccess) return e;
    if (is_empty(P)) return cudaSuccess;
    DeviceScope scope(stream);
    if (scope.status != cudaSuccess) return scope.status;
    const int dev = scope.device;
    key.call.force = g_tuning.force_kernel.load(std::memory_order_relaxed);
    key.call.tile_n = g_tuning.tile_n.load(std::memory_order_relaxed);
    key.call.stages = g_tuning.stages.load(std::memory_order_relaxed);
    key.call.max_ctas = g_tuning.max_ctas.load(std::memory_order_relaxed);
    key.call.split_k = g_tuning.split_k.load(std::memory_order_relaxed);
    key.call.device = dev;
    key.call.plan_epoch = g_plan_epoch.load(std::memory_order_relaxed);
    key.count = peerCount;
    key.multicast = multicastOut;
    for (int32_t i = 0; i < peerCount; ++i) {
        if (!peerOut[i]) return fail(cudaErrorInvalidValue, "srtMatmulAllGather: peerOut[%d] is null", i);
        key.peers[i] = peerOut[i];
    }
    if (!t_gather) t_gather.reset(new GatherEntry[kGatherCacheSize]);
    GatherEntry& ent = t_gather[hash_key(key.call) % kGatherCacheSize];
    if (!(ent.valid && memcmp(&ent.key, &key, sizeof key) == 0)) {
        ent.valid = false;
        Plan plan;
        e = plan_for(P, plan);
        if (e != cudaSuccess) return e;
        e = prepare_any(plan, ent.pr);
        if (e != cudaSuccess) return e;
        ent.fused = (plan.pub.kernel == srtMatmulKernelTcgen05Pair || plan.pub.kernel == srtMatmulKernelTcgen05) &&
                    ent.pr.splits <= 1 && ent.pr.gp.out_tma;
        if (ent.fused) {
            // the planner may have transposed the problem (column-order output): peers hold the same view
            memset(&ent.maps, 0, sizeof ent.maps);
            for (int32_t i = 0; i < peerCount && ent.fused; ++i)
                ent.fused = encode_out_map(&ent.maps.m[i], plan.Q, ent.pr.gp.ldo, peerOut[i]);
        }
        ent.pr.gp.n_peers = ent.fused ? (uint32_t)peerCount : 0u;
        ent.pr.gp.multicast = 0;
        if (multicastOut) {
            // 16-byte multimem stores: whole chunks only, and the multicast view aligned like the local one
            const bool ok = ent.fused && (plan.Q.N * plan.Q.elem) % 16 == 0 && reinterpret_cast<uintptr_t>(multicastOut) % 16 == 0;
            if (!ok)
                return fail(cudaErrorNotSupported,
                            "srtMatmulAllGatherMulticast: this product does not run on a 16-bit tensor-core kernel with a 16-byte "
                            "aligned, row-contiguous output whose row length is a multiple of 16 bytes; use srtMatmulAllGather");
            ent.maps.multicast = multicastOut;
            ent.pr.gp.multicast = 1;
        }
        ent.key = key;
        ent.valid = true;
    }
    if (!ent.fused) {
        e = launch_prepared(ent.pr, stream);
        if (e != cudaSuccess) return e;
        return copy_view_to_peers(P, oDesc, out, peerCount, peerOut, stream);
    }
    ent.pr.gp.wait_cycles = g_wait_limit_ns.load(std::memory_order_relaxed) * 2;
    const Prepared& pr = ent.pr;
    if (pr.kernel == srtMatmulKernelTcgen05Pair) {
        switch (pr.type) {
        case real32F: e = launch_pair_gather_bn<float>(pr.bn, pr.ma, pr.mb, pr.mo, pr.gp, pr.ctas, pr.smem, stream, ent.maps); break;
        case real16F: e = launch_pair_gather_bn<__half>(pr.bn, pr.ma, pr.mb, pr.mo, pr.gp, pr.ctas, pr.smem, stream, ent.maps); break;
        default: e = launch_pair_gather_bn<__nv_bfloat16>(pr.bn, pr.ma, pr.mb, pr.mo, pr.gp, pr.ctas, pr.smem, stream, ent.maps); break;
        }
    } else {
        switch (pr.type) {
        case real32F: e = launch_tc_gather_bn<float>(pr.bn, pr.ma, pr.mb, pr.mo, pr.gp, pr.ctas, pr.smem, stream, ent.maps); break;
        case real16F: e = launch_tc_gather_bn<__half>(pr.bn, pr.ma, pr.mb, pr.mo, pr.gp, pr.ctas, pr.smem, stream, ent.maps); break;
        default: e = launch_tc_gather_bn<__nv_bfloat16>(pr.bn, pr.ma, pr.mb, pr.mo, pr.gp, pr.ctas, pr.smem, stream, ent.maps); break;
        }
    }
    if (e == cudaSuccess) g_launches.fetch_add(1, std::memory_order_relaxed);
    return e;
}

cudaError_t srtMatmulAllGather(const void* a, const srtTensorDescriptor* aDesc, bool transA, const void* b,
                               const srtTensorDescriptor* bDesc, bool transB, const void* bias,
                               const srtTensorDescriptor* biasDesc, srtActivationType activation, void* out,
                               const srtTensorDescriptor* oDesc, int32_t peerCount, void* const* peerOut,
                               cudaStream_t stream)
{
    return gather_impl(a, aDesc, transA, b, bDesc, transB, bias, biasDesc, activation, out, oDesc, peerCount, peerOut, nullptr,
                       stream);
}

cudaError_t srtMatmulAllGatherMulticast(const void* a, const srtTensorDescriptor* aDesc, bool transA, const void* b,
                                        const srtTensorDescriptor* bDesc, bool transB, const void* bias,
                                        const srtTensorDescriptor* biasDesc, srtActivationType activation, void* out,
                                        const srtTensorDescriptor* oDesc, void* multicastOut, cudaStream_t stream)
{
    if (!multicastOut) return fail(cudaErrorInvalidValue, "srtMatmulAllGatherMulticast: null multicastOut");
    return gather_impl(a, aDesc, transA, b, bDesc, transB, bias, biasDesc, activation, out, oDesc, 0, nullptr, multicastOut, stream);
}

// ------------------------------------------------------------------ peer memory (one process per GPU)
// Device buffers that other processes of the same machine can map: plain cudaMalloc memory and
// CUDA IPC handles, no multicast objects.  The handle bytes travel over whatever channel the ranks
// already have (an MPI or torch.distributed all-gather of 64 bytes per rank).
cudaError_t srtPeerMemAlloc(size_t bytes, void** ptr, srtPeerMemHandle* handle)
{
    static_assert(sizeof(srtPeerMemHandle) == sizeof(cudaIpcMemHandle_t), "handle size");
    if (!ptr || !handle || bytes == 0) return fail(cudaErrorInvalidValue, "srtPeerMemAlloc: null argument or zero size");
    *ptr = nullptr;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) return fail(e, "srtPeerMemAlloc: cudaMalloc of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    cudaIpcMemHandle_t h;
    e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return fail(e, "srtPeerMemAlloc: cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
    }
    memcpy(handle->bytes, &h, sizeof h);
    *ptr = p;
    return cudaSuccess;
}

cudaError_t srtPeerMemOpen(const srtPeerMemHandle* handle, void** ptr)
{
    if (!ptr || !handle) return fail(cudaErrorInvalidValue, "srtPeerMemOpen: null argument");
    *ptr = nullptr;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle->bytes, sizeof h);
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail(e, "srtPeerMemOpen: cudaIpcOpenMemHandle failed: %s", cudaGetErrorString(e));
    *ptr = p;
    return cudaSuccess;
}

cudaError_t srtPeerSignal(void* const* peerFlags, int32_t peerCount, int32_t slot, uint64_t epoch, cudaStream_t stream)
{
    if (peerCount < 0 || peerCount >= kMaxFlagSlots || (peerCount > 0 && !peerFlags) || slot < 0 || slot >= kMaxFlagSlots)
        return fail(cudaErrorInvalidValue, "srtPeerSignal: at most %d peers, slot 0..%d", kMaxFlagSlots - 1, kMaxFlagSlots - 1);
    if (peerCount == 0) return cudaSuccess;
    DeviceScope scope(stream);
    if (scope.status != cudaSuccess) return scope.status;
    PeerSignalParams p;
    memset(&p, 0, sizeof p);
    for (int32_t i = 0; i < peerCount; ++i) {
        if (!peerFlags[i]) return fail(cudaErrorInvalidValue, "srtPeerSignal: peerFlags[%d] is null", i);
        p.peer_flags[i] = static_cast<unsigned long long*>(peerFlags[i]);
    }
    p.count = peerCount; p.slot = slot; p.epoch = epoch;
    peer_signal_kernel<<<1, 32, 0, stream>>>(p);
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) g_launches.fetch_add(1, std::memory_order_relaxed);
    return e;
}

cudaError_t srtPeerWait(const void* localFlags, int32_t slots, int32_t skipSlot, uint64_t epoch, uint64_t timeoutNs, cudaStream_t stream)
{
    if (!localFlags || slots < 1 || slots > kMaxFlagSlots)
        return fail(cudaErrorInvalidValue, "srtPeerWait: a flag array of 1..%d slots expected", kMaxFlagSlots);
    DeviceScope scope(stream);
    if (scope.status != cudaSuccess) return scope.status;
    const uint64_t ns = timeoutNs ? timeoutNs : (uint64_t)srt::kDefaultWaitLimitNs;
    peer_wait_kernel<<<1, 32, 0, stream>>>(static_cast<const volatile unsigned long long*>(localFlags), slots, skipSlot, epoch, ns * 2);
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) g_launches.fetch_add(1, std::memory_order_relaxed);
    return e;
}

cudaError_t srtPeerMemClose(void* ptr)
{
    if (!ptr) return cudaSuccess;
    cudaError_t e = cudaIpcCloseMemHandle(ptr);
    return e == cudaSuccess ? e : fail(e, "srtPeerMemClose: %s", cudaGetErrorString(e));
}

cudaError_t srtPeerMemFree(void* ptr)
{
    if (!ptr) return cudaSuccess;
    cudaError_t e = cudaFree(ptr);
    return e == cudaSuccess ? e : fail(e, "srtPeerMemFree: %s", cudaGetErrorString(e));
}

uint64_t srtMatmulLaunchCount(void) { return g_launches.load(); }

const char* srtMatmulGetLastErrorString(void) { return g_error; }

}  // extern "C"
