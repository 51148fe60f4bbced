// Thin inline-PTX wrappers for the sm_100a features the GEMM kernels use: mbarriers, TMA
// tile loads, tcgen05 tensor-memory allocation, MMA issue, commit and accumulator loads.
// Every wait is bounded: it gives up after a wall-clock limit and reports failure so that a
// broken pipeline ends the kernel with an error status instead of hanging the GPU.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace srt {

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// ----------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// arrive on the same-offset barrier of another CTA of the cluster (cta_rank), or of this one
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar, uint32_t cta_rank)
{
    asm volatile(
        "{\n\t.reg .b32 remote;\n\t"
        "mapa.shared::cluster.u32 remote, %0, %1;\n\t"
        "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [remote];\n\t}"
        ::"r"(bar), "r"(cta_rank) : "memory");
}

// The same with the default (CTA-scope release) semantics: the cluster-scope release above costs the
// arriving thread on the order of a thousand cycles, which matters when the arrive is issued once per
// pipeline stage.  For hand-offs whose data the async proxy reads (fence.proxy.async issued before).
__device__ __forceinline__ void mbar_arrive_remote(uint32_t bar, uint32_t cta_rank)
{
    asm volatile(
        "{\n\t.reg .b32 remote;\n\t"
        "mapa.shared::cluster.u32 remote, %0, %1;\n\t"
        "mbarrier.arrive.shared::cluster.b64 _, [remote];\n\t}"
        ::"r"(bar), "r"(cta_rank) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

// One try_wait with a suspend-time hint: the hardware parks the thread until the phase completes
// or the hint (in nanoseconds) runs out, so a waiting role does not spin on the issue ports that
// the epilogue warps need.
constexpr uint32_t kSuspendHintNs = 200000;

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(kSuspendHintNs)
        : "memory");
    return done != 0;
}

// cluster-scope acquire variant, for barriers that a peer CTA's MMA commit or arrive signals
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(kSuspendHintNs)
        : "memory");
    return done != 0;
}

// Limit of one pipeline wait.  A healthy wait lasts microseconds; the default limit is 2 s.  The
// kernels receive the limit as a parameter in SM clock cycles (GemmParams::wait_cycles: nanoseconds
// times 2, an upper bound of the cycles per nanosecond, so the limit is never shorter than asked) and
// measure with the SM's own cycle counter: reading %globaltimer costs about a microsecond, which put
// that microsecond on the critical path of every wait that did not succeed at its first try.
constexpr uint64_t kDefaultWaitLimitNs = 2000000000ull;

__device__ __forceinline__ uint64_t sm_clock()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%clock64;" : "=l"(t));
    return t;
}

// Waits for the phase with the given parity.  Returns false when the limit ran out or when another
// role of this CTA already gave up (*abort_flag != 0).  Each failed try_wait has already slept for up
// to kSuspendHintNs.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, uint64_t limit_cycles)
{
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = sm_clock();
    for (;;) {
        if (*abort_flag != 0) return false;
        if (sm_clock() - t0 > limit_cycles) return false;
        if (mbar_try_wait(bar, parity)) return true;          // parks for up to kSuspendHintNs
    }
}

__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, uint64_t limit_cycles)
{
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const uint64_t t0 = sm_clock();
    for (;;) {
        if (*abort_flag != 0) return false;
        if (sm_clock() - t0 > limit_cycles) return false;
        if (mbar_try_wait_cluster(bar, parity)) return true;          // parks for up to kSuspendHintNs
    }
}

// ----------------------------------------------------------------------------- TMA
__device__ __forceinline__ void prefetch_tensormap(const void* tmap)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// 3-D tiled load global -> shared of this CTA, completion counted in bytes on `bar`.
// c0 is the innermost coordinate: c0 * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* tmap, uint32_t bar,
                                            int32_t c0, int32_t c1, int32_t c2)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// 3-D tiled store shared -> global (bulk async group of the issuing thread).  Elements outside
// the tensor are not written, so ragged tile edges need no masking.
__device__ __forceinline__ void tma_store_3d(const void* tmap, uint32_t src, int32_t c0, int32_t c1, int32_t c2)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(src), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void bulk_commit_group()
{
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// waits until at most N of this thread's bulk groups still READ their shared-memory source
template <int N>
__device__ __forceinline__ void bulk_wait_group_read()
{
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// waits until at most N of this thread's bulk groups are incomplete (writes performed)
template <int N>
__device__ __forceinline__ void bulk_wait_group()
{
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// 16 bytes to every replica of a multicast (NVLS) mapping: the NVSwitch delivers the store to all
// GPUs bound to the multicast object, the issuing one included.  A plain bit copy, whatever the
// element type.
__device__ __forceinline__ void multimem_st_16(void* mc_ptr, const uint4& v)
{
    asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 ::"l"(mc_ptr), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
                   "f"(__uint_as_float(v.w)) : "memory");
}

// Programmatic dependent launch.  A kernel launched with the programmatic-stream-serialization
// attribute may be scheduled while its predecessor in the stream still runs, once every CTA of the
// predecessor has executed launch_dependents (or exited); it must execute grid_dependency_wait
// before touching anything the predecessor writes (the wait returns when the predecessor has
// completed and its writes are visible).  Both are no-ops in launches without the attribute.
__device__ __forceinline__ void launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Same load issued by one CTA of a cta_group::2 pair: the data lands in this CTA's shared
// memory, the byte count is signalled on `bar_cluster`, a shared::cluster address that may
// name the barrier of either CTA of the pair (see map_to_cta).  Not a multicast: one
// destination CTA.
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const void* tmap, uint32_t bar_cluster,
                                                 int32_t c0, int32_t c1, int32_t c2)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.cta_group::2"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// shared::cluster address of the same shared-memory offset in CTA `cta_rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t cta_rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta_rank));
    return r;
}

// a 32-bit store into the shared memory of CTA `cta_rank` of the cluster, at this CTA's offset `smem_addr`
__device__ __forceinline__ void st_shared_remote_u32(uint32_t smem_addr, uint32_t cta_rank, uint32_t value)
{
    asm volatile(
        "{\n\t.reg .b32 remote;\n\t"
        "mapa.shared::cluster.u32 remote, %0, %1;\n\t"
        "st.shared::cluster.u32 [remote], %2;\n\t}"
        ::"r"(smem_addr), "r"(cta_rank), "r"(value) : "memory");
}

__device__ __forceinline__ uint32_t ld_shared_remote_u32(uint32_t smem_addr, uint32_t cta_rank)
{
    uint32_t v;
    asm volatile(
        "{\n\t.reg .b32 remote;\n\t"
        "mapa.shared::cluster.u32 remote, %1, %2;\n\t"
        "ld.shared::cluster.u32 %0, [remote];\n\t}"
        : "=r"(v) : "r"(smem_addr), "r"(cta_rank) : "memory");
    return v;
}

// ----------------------------------------------------------------------------- tcgen05
__device__ __forceinline__ void tmem_alloc_cta1(uint32_t holder_smem, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(holder_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_cta1()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_cta1(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_alloc_cta2(uint32_t holder_smem, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(holder_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_cta2()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_cta2(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem desc] . B[smem desc]; 16-bit inputs (f16 / bf16 chosen by idesc)
__device__ __forceinline__ void umma_f16_cta1(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                              uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// fp32 inputs read as tf32 (the low 13 mantissa bits are ignored)
__device__ __forceinline__ void umma_tf32_cta1(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                               uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_f16_cta2(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                              uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_tf32_cta2(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                               uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// mbarrier arrives once all MMAs issued so far by this thread have completed
__device__ __forceinline__ void umma_commit_cta1(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(bar) : "memory");
}
// pair form: the same-offset barrier of every CTA named in cta_mask receives the arrive
__device__ __forceinline__ void umma_commit_cta2_mc(uint32_t bar, uint16_t cta_mask)
{
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64"
        " [%0], %1;"
        ::"r"(bar), "h"(cta_mask) : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives lane (base + i)
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
          "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
          "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]),
          "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]),
          "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// Same wait, tied to the destination registers of an earlier load: the compiler may not read
// (or move) them before this statement, which is when the hardware has written them.
__device__ __forceinline__ void tmem_ld_wait_regs(uint32_t (&v)[32])
{
    asm volatile(
        "tcgen05.wait::ld.sync.aligned;"
        : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]),
          "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15]),
          "+r"(v[16]), "+r"(v[17]), "+r"(v[18]), "+r"(v[19]), "+r"(v[20]), "+r"(v[21]), "+r"(v[22]), "+r"(v[23]),
          "+r"(v[24]), "+r"(v[25]), "+r"(v[26]), "+r"(v[27]), "+r"(v[28]), "+r"(v[29]), "+r"(v[30]), "+r"(v[31])
        :
        : "memory");
}

// The same for two loads in flight: both destination arrays are tied to the one wait.
__device__ __forceinline__ void tmem_ld_wait_regs2(uint32_t (&a)[32], uint32_t (&b)[32])
{
    asm volatile(
        "tcgen05.wait::ld.sync.aligned;"
        : "+r"(a[0]), "+r"(a[1]), "+r"(a[2]), "+r"(a[3]), "+r"(a[4]), "+r"(a[5]), "+r"(a[6]), "+r"(a[7]),
          "+r"(a[8]), "+r"(a[9]), "+r"(a[10]), "+r"(a[11]), "+r"(a[12]), "+r"(a[13]), "+r"(a[14]), "+r"(a[15]),
          "+r"(a[16]), "+r"(a[17]), "+r"(a[18]), "+r"(a[19]), "+r"(a[20]), "+r"(a[21]), "+r"(a[22]), "+r"(a[23]),
          "+r"(a[24]), "+r"(a[25]), "+r"(a[26]), "+r"(a[27]), "+r"(a[28]), "+r"(a[29]), "+r"(a[30]), "+r"(a[31])
        :
        : "memory");
    asm volatile(""
        : "+r"(b[0]), "+r"(b[1]), "+r"(b[2]), "+r"(b[3]), "+r"(b[4]), "+r"(b[5]), "+r"(b[6]), "+r"(b[7]),
          "+r"(b[8]), "+r"(b[9]), "+r"(b[10]), "+r"(b[11]), "+r"(b[12]), "+r"(b[13]), "+r"(b[14]), "+r"(b[15]),
          "+r"(b[16]), "+r"(b[17]), "+r"(b[18]), "+r"(b[19]), "+r"(b[20]), "+r"(b[21]), "+r"(b[22]), "+r"(b[23]),
          "+r"(b[24]), "+r"(b[25]), "+r"(b[26]), "+r"(b[27]), "+r"(b[28]), "+r"(b[29]), "+r"(b[30]), "+r"(b[31])
        :
        : "memory");
}

// ----------------------------------------------------------------------------- cluster
__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_arrive_release()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_acquire()
{
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

}  // namespace srt
