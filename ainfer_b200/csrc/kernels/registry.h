// Kernel registry: every device kernel is a __global__ function taking one
// POD argument struct by value. The registry records the struct's member
// offsets so that arguments can be set by index in member order, the
// convention of the reference's raw Level Zero loop
// (tools/decode/decode_l0.cpp:474-480: zeKernelSetArgumentValue by index).
#pragma once
#include <cstddef>
#include <cstdint>

namespace ainfer {

struct ArgField {
  uint32_t offset, size;
};

struct KernelDesc {
  const char *name;
  const void *fn;
  uint32_t args_size;
  const ArgField *fields;
  int nfields;
  int threads;          // threads per group (fixed)
  int items_per_group;  // work items one group covers; 0 = strides over any group count
  uint32_t smem_bytes;  // fixed dynamic shared memory (0 if none / static only)
  // optional: dynamic shared memory as a function of the argument bytes
  uint32_t (*smem_fn)(const void *args);
  // 1: blocks synchronise with each other, so the launch must be cooperative
  // (all groups co-resident) and the group count may not exceed what fits
  int cooperative;
  // 1: the kernel orders itself after its predecessor with griddepcontrol.wait, so a
  // command list may launch it early (programmatic dependency) to overlap its start-up
  int early_launch = 0;
};

void register_kernel(const KernelDesc &d);
int kernel_count();
const KernelDesc *kernel_at(int i);
const KernelDesc *kernel_find(const char *name);

// A translation unit whose kernels can report a stream fault registers a hook
// that stores the device address of the library's host-visible fault word in
// that unit's own __device__ pointer. Called once per device, device current.
typedef int (*FaultHook)(unsigned int *device_ptr);
void register_fault_hook(FaultHook h);
int fault_hook_count();
FaultHook fault_hook_at(int i);
struct FaultRegistrar {
  explicit FaultRegistrar(FaultHook h) { register_fault_hook(h); }
};

// Timeline builds only: every kernel translation unit registers a function that
// stores the address of the shared event buffer in that unit's own pointer.
typedef int (*TimelineHook)(unsigned long long *device_ptr);
void register_timeline_hook(TimelineHook h);
struct TimelineRegistrar {
  explicit TimelineRegistrar(TimelineHook h) { register_timeline_hook(h); }
};

// Marks an already registered kernel as safe to launch early (see KernelDesc::early_launch).
void mark_kernel_early_launch(const char *name);
struct EarlyLaunchMark {
  explicit EarlyLaunchMark(const char *name) { mark_kernel_early_launch(name); }
};

struct Registrar {
  explicit Registrar(const KernelDesc &d) { register_kernel(d); }
};

}  // namespace ainfer

#define AINFER_ARG(T, f) \
  { (uint32_t)offsetof(T, f), (uint32_t)sizeof(((T *)0)->f) }

// AINFER_REGISTER(Name, ArgsStruct, threads, items_per_group, smem_bytes, smem_fn, fields...)
#define AINFER_REGISTER(NAME, T, THREADS, ITEMS, SMEM, SMEMFN, ...)                          \
  static const ::ainfer::ArgField NAME##_fields[] = {__VA_ARGS__};                           \
  static ::ainfer::Registrar NAME##_registrar(::ainfer::KernelDesc{                          \
      #NAME, (const void *)NAME, (uint32_t)sizeof(T), NAME##_fields,                         \
      (int)(sizeof(NAME##_fields) / sizeof(NAME##_fields[0])), THREADS, ITEMS, SMEM, SMEMFN, 0})

#define AINFER_REGISTER_COOP(NAME, T, THREADS, ITEMS, SMEM, SMEMFN, ...)                     \
  static const ::ainfer::ArgField NAME##_fields[] = {__VA_ARGS__};                           \
  static ::ainfer::Registrar NAME##_registrar(::ainfer::KernelDesc{                          \
      #NAME, (const void *)NAME, (uint32_t)sizeof(T), NAME##_fields,                         \
      (int)(sizeof(NAME##_fields) / sizeof(NAME##_fields[0])), THREADS, ITEMS, SMEM, SMEMFN, 1})

// After AINFER_REGISTER(NAME, ...): the kernel calls pdl_wait() before it touches anything a
// predecessor writes (or that a predecessor still reads and it overwrites).
#define AINFER_EARLY_LAUNCH(NAME) static ::ainfer::EarlyLaunchMark NAME##_early(#NAME)
