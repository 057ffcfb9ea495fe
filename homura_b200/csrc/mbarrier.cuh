// mbarrier and bulk-copy (cp.async.bulk, no multicast) helpers shared by the kernels that run a
// producer/consumer ring in shared memory.  Every wait is bounded.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace hm {

constexpr unsigned long long MB_SPIN_LIMIT = 4000000ULL;  // polls before a wait gives up

__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mb_init(uint64_t* b, uint32_t n) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(b)), "r"(n) : "memory"); }
__device__ __forceinline__ void mb_arrive(uint64_t* b) { asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(s32(b)) : "memory"); }
__device__ __forceinline__ void mb_expect_tx(uint64_t* b, uint32_t bytes) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(s32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mb_try(uint64_t* b, uint32_t parity) {
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }" : "=r"(ok) : "r"(s32(b)), "r"(parity) : "memory");
    return ok != 0;
}
// The same poll with acquire semantics at cluster scope: for barriers completed by other CTAs' st.async stores.
__device__ __forceinline__ bool mb_try_cluster(uint64_t* b, uint32_t parity) {
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }" : "=r"(ok) : "r"(s32(b)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mb_wait_cluster(uint64_t* b, uint32_t parity, int* err, volatile int* abort_flag) {
    unsigned long long it = 0;
    while (!mb_try_cluster(b, parity)) {
        if (*abort_flag) return false;
        if (++it > MB_SPIN_LIMIT) {
            *abort_flag = 1;
            if (err) atomicExch(err, 2);
            return false;
        }
    }
    return true;
}
// Bounded wait; on overrun raises *err and returns false (callers skip the work that needed the data).
__device__ __forceinline__ bool mb_wait_limit(uint64_t* b, uint32_t parity, int* err, volatile int* abort_flag, unsigned long long limit) {
    unsigned long long it = 0;
    while (!mb_try(b, parity)) {
        if (*abort_flag) return false;
        if (++it > limit) {
            *abort_flag = 1;
            if (err) atomicExch(err, 2);
            return false;
        }
    }
    return true;
}
__device__ __forceinline__ bool mb_wait(uint64_t* b, uint32_t parity, int* err, volatile int* abort_flag) { return mb_wait_limit(b, parity, err, abort_flag, MB_SPIN_LIMIT); }
__device__ __forceinline__ void bulk_copy(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(s32(dst)), "l"(src), "r"(bytes), "r"(s32(bar)) : "memory");
}


}  // namespace hm
