// Thin inline-PTX wrappers used by every device header and kernel of this library.
// Everything here targets sm_100a only (NVIDIA B200): system-scope release/acquire
// accesses for cross-GPU signalling over NVLink, volatile vector accesses for LL packets,
// NVSwitch multimem (NVLS) loads/stores/reductions, mbarrier + bulk-copy (TMA) primitives.
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

#ifndef MSCCLPP_DEVICE_INLINE
#define MSCCLPP_DEVICE_INLINE __forceinline__ __device__
#endif
#ifndef MSCCLPP_HOST_DEVICE_INLINE
#define MSCCLPP_HOST_DEVICE_INLINE __forceinline__ __host__ __device__
#endif

#if defined(__CUDACC__)

namespace mscclpp {
namespace ptx {

// ------------------------------------------------------------------ timers / ids
MSCCLPP_DEVICE_INLINE uint64_t globaltimer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
MSCCLPP_DEVICE_INLINE uint32_t laneid() {
  uint32_t l;
  asm volatile("mov.u32 %0, %%laneid;" : "=r"(l));
  return l;
}
MSCCLPP_DEVICE_INLINE uint32_t smid() {
  uint32_t l;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(l));
  return l;
}
MSCCLPP_DEVICE_INLINE bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ------------------------------------------------------------------ scalar sys-scope accesses
MSCCLPP_DEVICE_INLINE uint64_t ld_acquire_sys(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
MSCCLPP_DEVICE_INLINE uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
MSCCLPP_DEVICE_INLINE uint64_t ld_relaxed_sys(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
MSCCLPP_DEVICE_INLINE uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
MSCCLPP_DEVICE_INLINE uint32_t ld_volatile(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
MSCCLPP_DEVICE_INLINE uint64_t ld_volatile(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
MSCCLPP_DEVICE_INLINE void st_release_sys(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
MSCCLPP_DEVICE_INLINE void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
MSCCLPP_DEVICE_INLINE void st_relaxed_sys(uint64_t* p, uint64_t v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
MSCCLPP_DEVICE_INLINE void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
MSCCLPP_DEVICE_INLINE void red_release_sys_add(uint64_t* p, uint64_t v) {
  asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
MSCCLPP_DEVICE_INLINE void red_relaxed_sys_add(uint64_t* p, uint64_t v) {
  asm volatile("red.relaxed.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
MSCCLPP_DEVICE_INLINE void red_release_gpu_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
MSCCLPP_DEVICE_INLINE uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
MSCCLPP_DEVICE_INLINE uint32_t atom_add_acqrel_gpu(uint32_t* p, uint32_t v) {
  uint32_t old;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}
MSCCLPP_DEVICE_INLINE void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
MSCCLPP_DEVICE_INLINE void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }
MSCCLPP_DEVICE_INLINE void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
MSCCLPP_DEVICE_INLINE void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ------------------------------------------------------------------ 16-byte vector accesses
// Bulk data movers (ld_nc_na_v4, st_na_v4, multimem 16-byte loads/stores) carry no "memory" clobber on
// purpose: the compiler may then keep many of them in flight; ordering against flags comes from the
// flag accesses themselves, which do clobber memory.
MSCCLPP_DEVICE_INLINE uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
MSCCLPP_DEVICE_INLINE void st_volatile_v4(void* p, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
MSCCLPP_DEVICE_INLINE uint2 ld_volatile_v2(const void* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
MSCCLPP_DEVICE_INLINE void st_volatile_v2(void* p, uint2 v) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}
// Streaming 16-byte load that bypasses L1 (peer memory is never cached coherently in L1).
MSCCLPP_DEVICE_INLINE uint4 ld_nc_na_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.relaxed.sys.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// Weak 16-byte loads for LOCAL memory. ld_cg_v4 reads through L2 only: for data that other SMs wrote during this launch
// and that was ordered by an acquire on a flag or counter. ld_input_v4 takes the non-coherent path without keeping the
// line: for kernel inputs that nothing writes during the launch. Both pipeline freely (the system-scope relaxed load
// above is a strong operation; a long run of them per thread was measured several times slower on local memory).
MSCCLPP_DEVICE_INLINE uint4 ld_cg_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
MSCCLPP_DEVICE_INLINE uint4 ld_input_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
MSCCLPP_DEVICE_INLINE void st_na_v4(void* p, uint4 v) {
  asm volatile("st.global.relaxed.sys.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w));
}

// ------------------------------------------------------------------ NVSwitch multimem (NVLS)
// `mc` is an address inside a CUDA multicast mapping: a load-reduce returns the element-wise
// reduction over every GPU bound to the mapping, a store is replicated to all of them.
MSCCLPP_DEVICE_INLINE uint4 multimem_ld_reduce_add_f16x2(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc));
  return v;
}
MSCCLPP_DEVICE_INLINE uint4 multimem_ld_reduce_add_bf16x2(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc));
  return v;
}
// bf16/f16 inputs summed with an fp32 accumulator inside the switch.
MSCCLPP_DEVICE_INLINE uint4 multimem_ld_reduce_add_f16x2_acc32(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc));
  return v;
}
MSCCLPP_DEVICE_INLINE uint4 multimem_ld_reduce_add_bf16x2_acc32(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc));
  return v;
}
MSCCLPP_DEVICE_INLINE uint4 multimem_ld_reduce_add_f32(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc));
  return v;
}
MSCCLPP_DEVICE_INLINE uint4 multimem_ld_reduce_min_f16x2(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.min.v4.f16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc));
  return v;
}
MSCCLPP_DEVICE_INLINE uint4 multimem_ld_reduce_min_bf16x2(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.min.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc));
  return v;
}
// fp8 reductions exist only on arch-specific Blackwell targets (sm_100a); accumulate in f16.
MSCCLPP_DEVICE_INLINE uint4 multimem_ld_reduce_add_e4m3x4(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f16.v4.e4m3x4 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc));
  return v;
}
MSCCLPP_DEVICE_INLINE uint4 multimem_ld_reduce_add_e5m2x4(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f16.v4.e5m2x4 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc));
  return v;
}
MSCCLPP_DEVICE_INLINE uint32_t multimem_ld_reduce_add_u32(const void* mc) {
  uint32_t v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.u32 %0, [%1];" : "=r"(v) : "l"(mc) : "memory");
  return v;
}
MSCCLPP_DEVICE_INLINE int32_t multimem_ld_reduce_add_s32(const void* mc) {
  int32_t v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.s32 %0, [%1];" : "=r"(v) : "l"(mc) : "memory");
  return v;
}
MSCCLPP_DEVICE_INLINE void multimem_st_v4(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w));
}
MSCCLPP_DEVICE_INLINE void multimem_st_v2(void* mc, uint2 v) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1,%2};" ::"l"(mc), "r"(v.x), "r"(v.y) : "memory");
}
MSCCLPP_DEVICE_INLINE void multimem_st_u32(void* mc, uint32_t v) {
  asm volatile("multimem.st.relaxed.sys.global.u32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}
MSCCLPP_DEVICE_INLINE void multimem_st_u64(void* mc, uint64_t v) {
  asm volatile("multimem.st.relaxed.sys.global.u64 [%0], %1;" ::"l"(mc), "l"(v) : "memory");
}
MSCCLPP_DEVICE_INLINE void multimem_red_add_f32x4(void* mc, uint4 v) {
  asm volatile("multimem.red.relaxed.sys.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
MSCCLPP_DEVICE_INLINE void multimem_red_add_bf16x2x4(void* mc, uint4 v) {
  asm volatile("multimem.red.relaxed.sys.global.add.v4.bf16x2 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
MSCCLPP_DEVICE_INLINE void multimem_red_add_f16x2x4(void* mc, uint4 v) {
  asm volatile("multimem.red.relaxed.sys.global.add.v4.f16x2 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
MSCCLPP_DEVICE_INLINE void multimem_red_release_add_u64(void* mc, uint64_t v) {
  asm volatile("multimem.red.release.sys.global.add.u64 [%0], %1;" ::"l"(mc), "l"(v) : "memory");
}
MSCCLPP_DEVICE_INLINE void multimem_red_relaxed_add_u64(void* mc, uint64_t v) {
  asm volatile("multimem.red.relaxed.sys.global.add.u64 [%0], %1;" ::"l"(mc), "l"(v) : "memory");
}
MSCCLPP_DEVICE_INLINE void multimem_red_release_add_u32(void* mc, uint32_t v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}

// ------------------------------------------------------------------ shared memory / mbarrier / bulk copies
MSCCLPP_DEVICE_INLINE uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

MSCCLPP_DEVICE_INLINE void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
MSCCLPP_DEVICE_INLINE void mbar_inval(uint64_t* bar) {
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
MSCCLPP_DEVICE_INLINE void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
MSCCLPP_DEVICE_INLINE void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
MSCCLPP_DEVICE_INLINE void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One non-blocking probe of the phase with the given parity; true once that phase has completed.
MSCCLPP_DEVICE_INLINE bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Untiled bulk copies. Both addresses 16-byte aligned, size a multiple of 16 bytes. No cluster
// multicast form is provided anywhere in this library: a remote tile is fetched by each CTA itself.
MSCCLPP_DEVICE_INLINE void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
MSCCLPP_DEVICE_INLINE void bulk_s2g(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst),
               "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}
MSCCLPP_DEVICE_INLINE void bulk_reduce_add_f32(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(gmem_dst),
               "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}
MSCCLPP_DEVICE_INLINE void bulk_reduce_add_bf16(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.noftz.bf16 [%0], [%1], %2;" ::"l"(gmem_dst),
               "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}
MSCCLPP_DEVICE_INLINE void bulk_reduce_add_f16(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.noftz.f16 [%0], [%1], %2;" ::"l"(gmem_dst),
               "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}
MSCCLPP_DEVICE_INLINE void bulk_reduce_add_u32(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.u32 [%0], [%1], %2;" ::"l"(gmem_dst),
               "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}
MSCCLPP_DEVICE_INLINE void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
MSCCLPP_DEVICE_INLINE void bulk_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
template <int N>
MSCCLPP_DEVICE_INLINE void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// Tiled (tensor-map) TMA copies, 2-D, never with cluster multicast.
MSCCLPP_DEVICE_INLINE void tma_load_2d(void* smem_dst, const void* tmap, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(smem_dst)),
      "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
MSCCLPP_DEVICE_INLINE void tma_load_2d_hint(void* smem_dst, const void* tmap, int x, int y, uint64_t* bar,
                                            uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, "
      "%3}], [%4], %5;" ::"r"(smem_u32(smem_dst)),
      "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}
MSCCLPP_DEVICE_INLINE void tma_store_2d(const void* tmap, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(tmap),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
MSCCLPP_DEVICE_INLINE void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ------------------------------------------------------------------ tcgen05 (5th-gen tensor core + TMEM)
MSCCLPP_DEVICE_INLINE void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
MSCCLPP_DEVICE_INLINE void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
MSCCLPP_DEVICE_INLINE void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
MSCCLPP_DEVICE_INLINE void tcgen05_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
MSCCLPP_DEVICE_INLINE void tcgen05_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// D[tmem] (+)= A[smem desc] * B[smem desc]; issued by ONE thread.
MSCCLPP_DEVICE_INLINE void tcgen05_mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Same, always accumulating (the predicate folds to "true": no register, no compare on the issue path).
MSCCLPP_DEVICE_INLINE void tcgen05_mma_f16_acc(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.eq.b32 p, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc)
      : "memory");
}
// Arrive (count 1) on a CTA-local mbarrier once all previously issued MMAs of this thread retire.
MSCCLPP_DEVICE_INLINE void tcgen05_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// Each thread of the warp reads 32 consecutive fp32 columns of its own TMEM lane.
MSCCLPP_DEVICE_INLINE void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
      "%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
MSCCLPP_DEVICE_INLINE void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- two-SM (cta_group::2) forms: a pair of CTAs of one cluster works on one MMA tile. The leader (cluster rank 0)
// issues the MMAs; both CTAs hold half of the operands and half of the accumulator rows.
MSCCLPP_DEVICE_INLINE uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the variable at `smemAddr` (a shared::cta address of this CTA) in CTA `rank` of the cluster.
MSCCLPP_DEVICE_INLINE uint32_t mapa_shared(uint32_t smemAddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smemAddr), "r"(rank));
  return r;
}
MSCCLPP_DEVICE_INLINE void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive (count 1) on an mbarrier of any CTA of the cluster, given its shared::cluster address.
MSCCLPP_DEVICE_INLINE void mbar_arrive_cluster(uint32_t clusterAddr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(clusterAddr) : "memory");
}
// Tiled load into THIS CTA's shared memory whose completion bytes are counted on an mbarrier given by its
// shared::cluster address (the pair leader's). No multicast: each CTA fetches its own half of the operands.
MSCCLPP_DEVICE_INLINE void tma_load_2d_pair(void* smem_dst, const void* tmap, int x, int y, uint32_t barClusterAddr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], "
      "[%4];" ::"r"(smem_u32(smem_dst)),
      "l"(tmap), "r"(x), "r"(y), "r"(barClusterAddr)
      : "memory");
}
MSCCLPP_DEVICE_INLINE void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
               : "memory");
}
MSCCLPP_DEVICE_INLINE void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
MSCCLPP_DEVICE_INLINE void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
MSCCLPP_DEVICE_INLINE void tcgen05_mma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
MSCCLPP_DEVICE_INLINE void tcgen05_mma_f16_pair_acc(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.eq.b32 p, 0, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc)
      : "memory");
}
// Arrive on the mbarrier at this offset in every CTA of `ctaMask` once the MMAs issued so far have retired.
MSCCLPP_DEVICE_INLINE void tcgen05_commit_pair(uint64_t* bar, uint16_t ctaMask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"(ctaMask)
               : "memory");
}

// Named barrier among `nthreads` threads of the CTA (ids 1..15; 0 is __syncthreads()).
MSCCLPP_DEVICE_INLINE void named_barrier(uint32_t id, uint32_t nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

}  // namespace ptx
}  // namespace mscclpp

#endif  // __CUDACC__
