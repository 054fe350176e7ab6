// C ABI for custom operators in shared libraries.
//
// A library exports
//     int ortb200_register_custom_ops(const ortb200_custom_op_api* api);
// and calls api->register_op(...) once per operator.  At run time the compute function receives its inputs and
// must fill its outputs through api->allocate_output.  Plays the part of the reference's OrtCustomOp /
// RegisterCustomOps entry point (onnxruntime/core/session/custom_ops.cc) with a much smaller surface.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ORTB200_CUSTOM_OP_API_VERSION 1

// ONNX TensorProto element type codes (1 = float, 7 = int64, 10 = float16, 16 = bfloat16, ...)
typedef struct {
  void* data;           // device or host pointer, see `on_gpu`
  int64_t dims[8];
  int32_t ndim;
  int32_t elem_type;
  int32_t on_gpu;       // 1: data lives on the CUDA device of the session
  int32_t present;      // 0: the optional input was omitted
} ortb200_tensor;

typedef struct ortb200_kernel_context ortb200_kernel_context;

typedef struct ortb200_custom_op_api {
  uint32_t version;
  // Attribute access for the node being computed; return 0 on success, non-zero when the attribute is absent.
  int (*attr_int)(const ortb200_kernel_context* ctx, const char* name, int64_t* out);
  int (*attr_float)(const ortb200_kernel_context* ctx, const char* name, float* out);
  int (*attr_string)(const ortb200_kernel_context* ctx, const char* name, char* out, int64_t capacity);
  // Creates output `index` with the given shape and type on the device of input 0 (host when there is none).
  int (*allocate_output)(ortb200_kernel_context* ctx, int index, const int64_t* dims, int ndim, int32_t elem_type,
                         ortb200_tensor* out);
  // CUDA stream of the run (null on the CPU provider).
  void* (*cuda_stream)(const ortb200_kernel_context* ctx);
  // compute: return 0 on success; on failure write a message with set_error and return non-zero
  void (*set_error)(ortb200_kernel_context* ctx, const char* message);
  int (*register_op)(const char* domain, const char* op_type,
                     int (*compute)(const struct ortb200_custom_op_api* api, ortb200_kernel_context* ctx,
                                    const ortb200_tensor* inputs, int num_inputs, int num_outputs, void* user),
                     void* user);
} ortb200_custom_op_api;

#ifdef __cplusplus
}
#endif
