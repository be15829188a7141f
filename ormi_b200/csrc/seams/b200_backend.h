// Additive surface of the B200 backend for C++ code above ormi-core (the reference has no counterpart: it drives
// device 0 only, ormi-core/csrc/backend/cuda/allocator.cu:22, jit.cu:17, and has no collectives).
//
//   set_active_device  the device later allocations go to, and with them the graphs built on those tensors; one process
//                      per GPU calls it once with its local rank.  Throws std::runtime_error when there is no such device.
//   b200_context       the backend context of a device (-1: the active one), for the entry points of ormi_b200.h that
//                      ormi-core's own API has no word for: ormi_b200_comm_init / ormi_b200_allreduce_sum_f32 on the
//                      `ptr` of realized Buffers (the gradient all-reduce of a batch-sharded step), ormi_b200_set_option,
//                      the asynchronous copies.
#pragma once
#include "ormi_b200.h"

namespace ormi::cuda {
void set_active_device(int device);
int active_device();
ormi_b200_ctx* b200_context(int device = -1);
}  // namespace ormi::cuda
