/* C API of the onnxruntime_b200 runtime: load a model, run it, read the outputs - from C, C++ or any language with a
 * C foreign-function interface, without Python.  Link with lib/libortb200.so.
 *
 * The shape follows the reference's C API (include/onnxruntime/core/session/onnxruntime_c_api.h: CreateSession,
 * SessionGetInputCount / SessionGetInputName, CreateTensorWithDataAsOrtValue, Run, GetTensorMutableData,
 * GetTensorTypeAndShape, Release*), reduced to plain functions instead of a versioned function table.
 *
 * Every function returns 0 on success; otherwise a non-zero code of the OrtErrorCode numbering (1 FAIL,
 * 2 INVALID_ARGUMENT, 3 NO_SUCHFILE, 6 RUNTIME_EXCEPTION, 9 NOT_IMPLEMENTED, 10 INVALID_GRAPH, 11 EP_FAIL) and
 * ortb200_last_error() returns the message (per thread). */
#ifndef ORTB200_C_API_H_
#define ORTB200_C_API_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ortb200_session ortb200_session;
typedef struct ortb200_value ortb200_value;

/* A tensor the caller owns (inputs) or a view of a tensor the runtime owns (outputs).  elem_type uses the ONNX
 * TensorProto numbering (1 float, 6 int32, 7 int64, 10 float16, 16 bfloat16, ...).  device_type: 0 host, 1 CUDA. */
typedef struct {
  void* data;
  int32_t elem_type;
  int32_t ndim;
  int64_t dims[8];
  int32_t device_type;
  int32_t device_id;
} ortb200_tensor_view;

const char* ortb200_last_error(void);
const char* ortb200_version(void);

/* model_path, or model_bytes / model_size when model_path is NULL.  provider: "CPUExecutionProvider" or
 * "CUDAExecutionProvider".  config: NULL or a NULL-terminated list key, value, key, value, ... of session config
 * entries and of the option names "graph_optimization_level", "enable_profiling", "logid", "log_severity_level",
 * "enable_cuda_graph". */
int ortb200_create_session(const char* model_path, const void* model_bytes, size_t model_size, const char* provider,
                           int device_id, const char* const* config, ortb200_session** out);
void ortb200_release_session(ortb200_session* session);

int ortb200_session_input_count(const ortb200_session* session, size_t* out);
int ortb200_session_output_count(const ortb200_session* session, size_t* out);
/* The returned strings live as long as the session. */
int ortb200_session_input_name(const ortb200_session* session, size_t index, const char** out);
int ortb200_session_output_name(const ortb200_session* session, size_t index, const char** out);

/* Runs the model.  inputs[i] describes memory that must stay valid during the call (it is wrapped, not copied, when it
 * already lives where the model wants it).  output_names may be NULL (all outputs, in model order; num_outputs must
 * then equal the output count).  outputs[i] receives a value to release with ortb200_release_value. */
int ortb200_run(ortb200_session* session, const char* const* input_names, const ortb200_tensor_view* inputs,
                size_t num_inputs, const char* const* output_names, size_t num_outputs, ortb200_value** outputs);

/* View of an output; the memory belongs to the value.  host = 1 first copies a device tensor to host memory. */
int ortb200_value_tensor(ortb200_value* value, int host, ortb200_tensor_view* out);
void ortb200_release_value(ortb200_value* value);

/* Ends profiling (SessionOptions enable_profiling) and returns the trace file's path (valid until the next call). */
int ortb200_end_profiling(ortb200_session* session, const char** out_path);

#ifdef __cplusplus
}
#endif
#endif /* ORTB200_C_API_H_ */
