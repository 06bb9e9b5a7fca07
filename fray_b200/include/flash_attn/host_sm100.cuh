#pragma once
// Host-side helpers shared by the sm_100a attention launchers: argument validation,
// return codes, TMA tensor-map construction (driver entry point resolved at run time so
// the generated library needs no link-time libcuda) and device status readback.

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "sm100_ptx.cuh"

namespace fray {

// Values written to `__return_code` by the launchers. 0 means the kernel was queued.
enum AttnReturnCode : int {
  kAttnOk = 0,
  kAttnBadShape = 1,        // a count is not positive, batch * heads exceeds 65535, K/V heads do not divide the
                            // query heads, or the softmax scale is not positive and finite
  kAttnBadPointer = 2,      // null or not 16-byte aligned
  kAttnBadStride = 3,       // a stride is not a positive multiple of 8 elements (16 bytes)
  kAttnNoDriverEntry = 5,   // cuTensorMapEncodeTiled could not be resolved
  kAttnTensorMapFailed = 6, // the driver rejected the tensor map (layout not expressible)
  kAttnSmemAttrFailed = 7,  // cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed
  kAttnLaunchFailed = 8,    // the launch itself reported an error
};

// Element strides of one [B,H,S,D] tensor; the D stride is 1 by contract.
struct AttnStrides {
  int64_t b, h, s;
};

struct AttnShape {
  int B, H, S, D;
};

// Optional features.  kv_group: query heads per K/V head (1 = every query head has its own K/V;
// g > 1 = grouped-query attention, K and V hold H / g heads and query head h reads K/V head h / g).
// lse: when not null, receives log(sum_j exp(scale * q.k_j)) per query row as fp32 [B, H, S], contiguous.
// seq_k: number of keys (K/V rows); the shape's S is the number of queries.  With a causal mask and
// seq_k != S, query i sees keys 0..i (the mask is aligned to the top left corner, as in torch attention).
struct AttnExtras {
  int kv_group;
  float* lse;
  int seq_k;
};

// shp describes Q and O, shp_kv K and V (their own head count and length).  Strides of modes of
// extent 1 are ignored.
inline int validate_attn_args(const void* q, const void* k, const void* v, const void* o, const AttnShape& shp,
                              const AttnShape& shp_kv, const AttnStrides (&st)[4]) {
  if (shp.B <= 0 || shp.H <= 0 || shp.S <= 0 || shp_kv.H <= 0 || shp_kv.S <= 0) return kAttnBadShape;
  if (static_cast<int64_t>(shp.B) * shp.H > 65535) return kAttnBadShape;  // batch * heads is a grid dimension
  const void* ptrs[4] = {q, k, v, o};
  for (int i = 0; i < 4; ++i) {
    if (ptrs[i] == nullptr || (reinterpret_cast<uintptr_t>(ptrs[i]) & 15u) != 0) return kAttnBadPointer;
    const AttnShape& e = (i == 1 || i == 2) ? shp_kv : shp;
    const int64_t s3[3] = {st[i].b, st[i].h, st[i].s};
    const int extent[3] = {e.B, e.H, e.S};
    for (int d = 0; d < 3; ++d) {
      if (extent[d] > 1 && (s3[d] <= 0 || (s3[d] & 7) != 0)) return kAttnBadStride;
    }
  }
  return kAttnOk;
}

using PFN_encodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                     const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                     CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline PFN_encodeTiled get_encode_tiled() {
  static PFN_encodeTiled fn = []() -> PFN_encodeTiled {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    return reinterpret_cast<PFN_encodeTiled>(p);
  }();
  return fn;
}

// Tensor map over a 16-bit (fp16 or bf16, see operand_t) [B,H,S,D] tensor (D contiguous) whose box is
// `box_rows` sequence positions x 64 head-dim elements (one 128-byte swizzle span).
inline int make_attn_tensor_map(CUtensorMap* map, const void* base, const AttnShape& shp, const AttnStrides& st,
                                int box_rows) {
  PFN_encodeTiled enc = get_encode_tiled();
  if (enc == nullptr) return kAttnNoDriverEntry;
  // A size-1 mode never advances, so any legal (16-byte multiple) stride will do.
  const int64_t sb = shp.B > 1 ? st.b : static_cast<int64_t>(shp.D);
  const int64_t sh = shp.H > 1 ? st.h : static_cast<int64_t>(shp.D);
  const int64_t ss = shp.S > 1 ? st.s : static_cast<int64_t>(shp.D);
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(shp.D), static_cast<cuuint64_t>(shp.S),
                        static_cast<cuuint64_t>(shp.H), static_cast<cuuint64_t>(shp.B)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(ss) * 2, static_cast<cuuint64_t>(sh) * 2,
                           static_cast<cuuint64_t>(sb) * 2};
  cuuint32_t box[4] = {64u, static_cast<cuuint32_t>(box_rows), 1u, 1u};
  cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  CUresult r = enc(map, kOperandIsBf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? kAttnOk : kAttnTensorMapFailed;
}

// Same as make_attn_tensor_map, but remembers the last few encodings per host thread: a caller that
// launches on the same buffers again (the common case: a fixed set of activations per layer, or a
// benchmark loop) skips the driver call.  A tensor map depends only on the key compared below.
inline int cached_attn_tensor_map(CUtensorMap* map, const void* base, const AttnShape& shp, const AttnStrides& st,
                                  int box_rows) {
  struct Entry {
    const void* base = nullptr;
    AttnShape shp{0, 0, 0, 0};
    AttnStrides st{0, 0, 0};
    int box_rows = 0;
    CUtensorMap map;
  };
  constexpr int kEntries = 16;
  thread_local Entry cache[kEntries];
  thread_local int next = 0;
  for (int e = 0; e < kEntries; ++e) {
    const Entry& c = cache[e];
    if (c.base == base && c.box_rows == box_rows && c.shp.B == shp.B && c.shp.H == shp.H && c.shp.S == shp.S &&
        c.shp.D == shp.D && c.st.b == st.b && c.st.h == st.h && c.st.s == st.s) {
      *map = c.map;
      return kAttnOk;
    }
  }
  const int rc = make_attn_tensor_map(map, base, shp, st, box_rows);
  if (rc == kAttnOk) {
    Entry& c = cache[next];
    next = (next + 1) % kEntries;
    c.base = base;
    c.shp = shp;
    c.st = st;
    c.box_rows = box_rows;
    c.map = *map;
  }
  return rc;
}

// Raises a kernel's dynamic shared-memory limit once per device of this process (function
// attributes are per device; the reference sets the attribute on every launch,
// fray/include/flash_attn/flashattn_cute.cuh:231).  Tag makes the bookkeeping unique per kernel
// configuration: kernels of equal signature share a function-pointer type.
// regs_after_setmaxnreg: for kernels whose warps re-balance registers with setmaxnreg, the sum of
// the budgets over all threads.  setmaxnreg.inc draws from the CTA's allocation at launch (threads x
// registers per thread as compiled) and blocks without bound if that pool cannot cover it, so a
// kernel compiled with fewer registers than its budgets assume is refused here instead.
template <class Tag, class Kernel>
inline int ensure_dynamic_smem(Kernel kernel, int bytes, int threads = 0, int regs_after_setmaxnreg = 0) {
  constexpr int kMaxDevices = 64;
  static bool done[kMaxDevices] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return kAttnSmemAttrFailed;
  }
  const bool tracked = dev >= 0 && dev < kMaxDevices;
  if (tracked && done[dev]) return kAttnOk;
  if (regs_after_setmaxnreg > 0) {
    cudaFuncAttributes attr;
    if (cudaFuncGetAttributes(&attr, kernel) != cudaSuccess) {
      (void)cudaGetLastError();
      return kAttnLaunchFailed;
    }
    if (attr.numRegs * threads < regs_after_setmaxnreg) return kAttnLaunchFailed;
  }
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) {
    (void)cudaGetLastError();
    return kAttnSmemAttrFailed;
  }
  if (tracked) done[dev] = true;
  return kAttnOk;
}

// Order in which the query tiles of a causal problem start: slice by slice (CTAs side by side share a slice's
// K and V in L2), or the heaviest tiles of ALL (batch, head) slices first, which lets the hardware's
// first-come scheduling even out the tiles' unequal lengths.  Measured on 4096- and 16384-row causal problems,
// heaviest first gains 7-45 % while there are at most seven rounds of CTAs (K and V up to 134 MB) and is level
// or slightly behind at fourteen rounds (256 MB: K and V of the slices in flight no longer share L2); at 1024
// and 2048 rows, where a slice's few tiles run side by side anyway, it loses up to 13 %.
static constexpr long long kHeaviestFirstMaxKvBytes = 160LL * 1000 * 1000;
static constexpr int kHeaviestFirstMinRows = 4096;
// The same decision as a group size for kernels whose grid is (slice inside its group, tiles, groups): all
// slices in one group, or 0 for slice by slice.  (Several groups of slices that each stay under the limit were
// measured on the 256 MB configurations: no difference from slice by slice within the run-to-run spread.)
inline int heaviest_first_group(bool causal, const AttnShape& shp, const AttnShape& shp_kv);
inline bool heaviest_first_order(bool causal, const AttnShape& shp, const AttnShape& shp_kv) {
  const long long kv_bytes = 2LL * shp_kv.B * shp_kv.H * shp_kv.S * shp_kv.D * 2;
  return causal && shp.S >= kHeaviestFirstMinRows && kv_bytes <= kHeaviestFirstMaxKvBytes;
}
inline int heaviest_first_group(bool causal, const AttnShape& shp, const AttnShape& shp_kv) {
  return heaviest_first_order(causal, shp, shp_kv) ? shp.B * shp.H : 0;
}

// Number of SMs of the current device (cached per device of this process); 0 on failure.
inline int device_sm_count() {
  constexpr int kMaxDevices = 64;
  static int count[kMaxDevices] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  if (dev >= 0 && dev < kMaxDevices && count[dev] > 0) return count[dev];
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  if (dev >= 0 && dev < kMaxDevices) count[dev] = n;
  return n;
}

// Synchronising read of the sticky device status words; clears them when asked.
inline int read_attn_status(int* out4, bool clear) {
  int host[4] = {0, 0, 0, 0};
  cudaError_t e = cudaMemcpyFromSymbol(host, sm100::fray_attn_status, sizeof(host));
  if (e != cudaSuccess) return static_cast<int>(e);
  for (int i = 0; i < 4; ++i) out4[i] = host[i];
  if (clear && host[0] != 0) {
    int zero[4] = {0, 0, 0, 0};
    e = cudaMemcpyToSymbol(sm100::fray_attn_status, zero, sizeof(zero));
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  return 0;
}

}  // namespace fray
