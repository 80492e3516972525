// Launch accounting: a process-wide count of kernel launches and, when switched on, CUDA-event
// timing of every launch grouped by "slot" (which step of the layer the launch belongs to).
// Events are recorded on the launch stream, so the figures are device times of the kernels
// as they ran inside the caller's timed region.  Host-side state only; nothing is allocated on
// the device.
#pragma once

#include <cuda_runtime.h>

namespace mok {

enum ProfSlot : int {
    kSlotScheduler = 0, kSlotQuantize, kSlotAllGather, kSlotBarrier, kSlotEpilogue,
    kSlotDispatch, kSlotCombine,
    kSlotGateUpShared, kSlotDownShared, kSlotGateUpRouted, kSlotDownRouted,
    kSlotDgradDownShared, kSlotDgradGateUpShared, kSlotWgradShared,
    kSlotDgradDownRouted, kSlotDgradGateUpRouted, kSlotWgradRouted,
    kSlotGemmTest, kSlotOther,
    kNumSlots
};

void prof_begin(int slot, cudaStream_t stream, int kernels);
void prof_end(int slot, cudaStream_t stream);

struct ProfScope {
    int slot;
    cudaStream_t stream;
    ProfScope(int s, cudaStream_t st, int kernels = 1) : slot(s), stream(st) { prof_begin(slot, stream, kernels); }
    ~ProfScope() { prof_end(slot, stream); }
};

}  // namespace mok
