// Launches with programmatic dependent launch: a kernel launched this way may
// start while its predecessor in the stream is still running.  Every kernel of
// this package follows one discipline, which makes that safe:
//   - work that does not depend on earlier kernels (fetching weights) may come
//     first;
//   - pdl_wait() before the first read of anything an earlier kernel wrote and
//     before the first write to global memory.  It returns when the
//     predecessor has completed and its writes are visible.  Since every
//     kernel waits before it completes, completion is transitive along the
//     stream;
//   - pdl_trigger() right after the wait: the next kernel in the stream may be
//     scheduled once every block of this one has passed its wait.  Triggering
//     before the wait would let the whole chain of future kernels become
//     resident at once, each waiting on the one before and taking the
//     processors from the one that runs (measured: a decode step 40% slower);
//     after the wait, exactly one kernel runs ahead.
// Decode steps are chains of many short kernels; overlapping each kernel's
// launch and first memory round trip with its predecessor's tail is worth a
// large part of the step time.  ALPACCA_B200_PDL=0 turns the attribute off
// (the device-side instructions are then no-ops).
#pragma once
#include <cuda_runtime.h>
#include <stdlib.h>

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

static inline bool ab_pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("ALPACCA_B200_PDL");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on == 1;
}

// One kind of kernel must not start early: the one that follows a kernel with another split of the SM's
// memory between shared memory and L1 (the product after the decode attention, which fills shared
// memory).  Started while such a kernel still runs, it and the chain of dependents behind it lost
// 0.4 to 50 microseconds per layer, the more the larger the model (measured at widths 2048 to 4096);
// started after it, nothing.  The host holds dependent launch for that one launch.
static int ab_pdl_held = 0;
extern "C" __attribute__((visibility("default"))) void ab_pdl_hold(int hold) { ab_pdl_held = hold ? 1 : 0; }

template <typename... KArgs, typename... Args>
static inline cudaError_t ab_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (ab_pdl_enabled() && !ab_pdl_held) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
