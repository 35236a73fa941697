// Building blocks for kernels on the fifth-generation tensor cores: mbarriers with
// bounded waits, TMA tile loads and tensor maps, shared-memory matrix descriptors for the
// 128-byte swizzle, tcgen05 MMA / commit / tensor-memory load and store.
#pragma once
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace bw {

#ifndef SHRIKE_WAIT_HINT_NS
#define SHRIKE_WAIT_HINT_NS 20000
#endif
constexpr unsigned WAIT_HINT_NS = SHRIKE_WAIT_HINT_NS;   // one try_wait may sleep this long
constexpr unsigned WAIT_LIMIT = 2000000000u / (WAIT_HINT_NS < 100 ? 100 : WAIT_HINT_NS);   // tries before a wait gives up: about two seconds

__device__ __forceinline__ unsigned smem_u32(const void* p) { return static_cast<unsigned>(__cvta_generic_to_shared(p)); }

// ---- mbarriers
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(WAIT_HINT_NS) : "memory");
  return ok != 0;
}
// One look at the barrier without suspending: about 15 clocks, against 50 for a try_wait with a time hint.
__device__ __forceinline__ bool mbar_test_wait(unsigned long long* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Waits for the phase with the given parity.  Returns false when the wait ran out (the
// caller's code `who` goes to *status, *abort is raised) or when another role raised *abort.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity, volatile int* abort, int* status, int who) {
  if (mbar_test_wait(bar, parity)) return true;   // the usual case in a pipeline that runs ahead
  for (unsigned tries = 0; tries < WAIT_LIMIT; ++tries) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort) return false;
  }
  *abort = 1;
  if (status != nullptr && *status == 0) *status = who;
  return false;
}

// ---- TMA
__device__ __forceinline__ void tma_load_2d(void* smem, const CUtensorMap* map, unsigned long long* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem)), "l"(reinterpret_cast<unsigned long long>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
// Makes shared-memory writes of this thread visible to the asynchronous proxy (TMA, MMA).
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- tcgen05
__device__ __forceinline__ void tmem_alloc(unsigned* slot_in_smem, unsigned columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot_in_smem)), "r"(columns) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free(unsigned address, unsigned columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Matrix descriptor of an operand tile in the 128-byte swizzle (rows of 64 bf16, 8-row
// groups 1024 bytes apart).  K-major: `leading` is unused (1).  MN-major: `leading_bytes` is
// the distance between 64-element groups along M/N, `stride_bytes` between 8-row groups
// along K.
__device__ __forceinline__ unsigned long long smem_descriptor(unsigned addr, unsigned leading_bytes = 16, unsigned stride_bytes = 1024) {
  return static_cast<unsigned long long>((addr & 0x3FFFFu) >> 4) | (static_cast<unsigned long long>(leading_bytes >> 4) << 16) |
         (static_cast<unsigned long long>(stride_bytes >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// kind::f16 instruction descriptor: D float32, A and B bfloat16, A K-major; B K-major or MN-major.
__device__ __forceinline__ unsigned instruction_descriptor(int m, int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | (static_cast<unsigned>(n >> 3) << 17) |
         (static_cast<unsigned>(m >> 4) << 24);
}
__device__ __forceinline__ void umma(unsigned tmem_d, unsigned long long a, unsigned long long b, unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 lanes x 32 columns of 32-bit: thread i of the warp gets lane (quarter * 32 + i), columns c .. c + 31.
__device__ __forceinline__ void tmem_load32(unsigned taddr, unsigned (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_store32(unsigned taddr, const unsigned (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_load() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_store() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---- tensor maps (host)
using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiled encode_tiled() {
  static EncodeTiled fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiled>(ptr);
  });
  return fn;
}

struct MapKey {
  const void* base;
  long long rows;
  int cols, box_rows;
  bool operator==(const MapKey& o) const { return base == o.base && rows == o.rows && cols == o.cols && box_rows == o.box_rows; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.base);
    h = h * 1000003u ^ static_cast<size_t>(k.rows);
    h = h * 1000003u ^ static_cast<size_t>(k.cols);
    return h * 1000003u ^ static_cast<size_t>(k.box_rows);
  }
};

// A row-major [rows, cols] bfloat16 matrix seen as boxes of box_rows x 64 elements in the
// 128-byte swizzle; out-of-range parts of a box read as zero.  cols must be a multiple of 8.
static inline int tensor_map_bf16(const void* base, long long rows, int cols, int box_rows, CUtensorMap* out) {
  static std::mutex mutex;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{base, rows, cols, box_rows};
  std::lock_guard<std::mutex> guard(mutex);
  auto found = cache.find(key);
  if (found != cache.end()) {
    *out = found->second;
    return SHRIKE_OK;
  }
  EncodeTiled encode = encode_tiled();
  if (encode == nullptr || cols % 8 || box_rows < 1 || box_rows > 256) return SHRIKE_BAD_ARGUMENT;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t element_strides[2] = {1, 1};
  CUtensorMap map;
  const CUresult rc = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                             element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return 1000 + static_cast<int>(rc);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, map);
  *out = map;
  return SHRIKE_OK;
}

}  // namespace bw
