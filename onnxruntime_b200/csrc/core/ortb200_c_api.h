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

/* ---------------------------------------------------------------------------------------------------------------
 * Wider surface: option objects, type information, model metadata, I/O binding, runtime-owned tensors, environment.
 * Counterparts in the reference's table: CreateSessionOptions / SetSessionGraphOptimizationLevel / SetIntraOpNumThreads /
 * AddSessionConfigEntry / SessionOptionsAppendExecutionProvider / RegisterCustomOpsLibrary, CreateRunOptions /
 * RunOptionsSetTerminate, SessionGetInputTypeInfo, SessionGetModelMetadata / ModelMetadataLookupCustomMetadataMap,
 * CreateIoBinding / BindInput / BindOutput / BindOutputToDevice / RunWithBinding / GetBoundOutputValues,
 * CreateTensorAsOrtValue, GetAvailableProviders. */
typedef struct ortb200_session_options ortb200_session_options;
typedef struct ortb200_run_options ortb200_run_options;
typedef struct ortb200_io_binding ortb200_io_binding;

int ortb200_create_session_options(ortb200_session_options** out);
void ortb200_release_session_options(ortb200_session_options* options);
int ortb200_session_options_set_graph_optimization_level(ortb200_session_options* options, int level); /* 0, 1, 2, 99 */
int ortb200_session_options_set_intra_op_num_threads(ortb200_session_options* options, int n);
int ortb200_session_options_set_inter_op_num_threads(ortb200_session_options* options, int n);
int ortb200_session_options_set_execution_mode(ortb200_session_options* options, int mode);            /* 0 sequential, 1 parallel */
int ortb200_session_options_set_log_id(ortb200_session_options* options, const char* logid);
int ortb200_session_options_set_log_severity_level(ortb200_session_options* options, int level);
int ortb200_session_options_enable_profiling(ortb200_session_options* options, const char* file_prefix);
int ortb200_session_options_set_optimized_model_filepath(ortb200_session_options* options, const char* path);
int ortb200_session_options_add_config_entry(ortb200_session_options* options, const char* key, const char* value);
int ortb200_session_options_add_free_dimension_override_by_name(ortb200_session_options* options, const char* name, int64_t value);
/* provider: "CUDAExecutionProvider" or "CPUExecutionProvider"; keys / values: num_options provider options
 * ("device_id", "enable_cuda_graph", ...).  Providers are tried in the order they were appended; CPU is always last. */
int ortb200_session_options_append_execution_provider(ortb200_session_options* options, const char* provider,
                                                      const char* const* keys, const char* const* values, size_t num_options);
/* Loads a shared library that exports the custom-operator registration entry point (custom_op_api.h). */
int ortb200_session_options_register_custom_ops_library(ortb200_session_options* options, const char* path);
int ortb200_create_session_from_options(const char* model_path, const void* model_bytes, size_t model_size,
                                        const ortb200_session_options* options, ortb200_session** out);

int ortb200_create_run_options(ortb200_run_options** out);
void ortb200_release_run_options(ortb200_run_options* options);
int ortb200_run_options_set_tag(ortb200_run_options* options, const char* tag);
int ortb200_run_options_set_log_severity_level(ortb200_run_options* options, int level);
int ortb200_run_options_add_config_entry(ortb200_run_options* options, const char* key, const char* value);
int ortb200_run_options_set_terminate(ortb200_run_options* options, int terminate); /* may be called from another thread */
int ortb200_run_with_options(ortb200_session* session, const ortb200_run_options* options, const char* const* input_names,
                             const ortb200_tensor_view* inputs, size_t num_inputs, const char* const* output_names,
                             size_t num_outputs, ortb200_value** outputs);

/* Declared type of a graph input / output.  dims[i] is -1 for a symbolic or unknown dimension, and dim_params[i] (when
 * dim_params is not NULL) then points to the symbol's name or to "".  has_shape = 0 means the rank is unknown. */
typedef struct {
  int32_t elem_type;
  int32_t has_shape;
  int32_t ndim;
  int64_t dims[8];
  const char* dim_params[8];
} ortb200_type_info;
int ortb200_session_input_type_info(const ortb200_session* session, size_t index, ortb200_type_info* out);
int ortb200_session_output_type_info(const ortb200_session* session, size_t index, ortb200_type_info* out);
int ortb200_session_overridable_initializer_count(const ortb200_session* session, size_t* out);
int ortb200_session_overridable_initializer_name(const ortb200_session* session, size_t index, const char** out);

/* Model metadata; strings live as long as the session. */
typedef struct {
  const char* producer_name;
  const char* graph_name;
  const char* domain;
  const char* description;
  int64_t version;
  size_t num_custom_keys;
} ortb200_model_metadata;
int ortb200_session_model_metadata(const ortb200_session* session, ortb200_model_metadata* out);
int ortb200_session_custom_metadata_key(const ortb200_session* session, size_t index, const char** key);
/* *value is NULL when the key is absent. */
int ortb200_session_lookup_custom_metadata(const ortb200_session* session, const char* key, const char** value);
int ortb200_session_provider_count(const ortb200_session* session, size_t* out);
int ortb200_session_provider_name(const ortb200_session* session, size_t index, const char** out);
int ortb200_session_profiling_start_time_ns(const ortb200_session* session, int64_t* out);
/* Turns a device-side timeout or argument error recorded by a kernel into an error code (see check_device_status). */
int ortb200_session_check_device_status(ortb200_session* session);

/* I/O binding: inputs and outputs stay where they are bound (no copies through the host). */
int ortb200_create_io_binding(ortb200_session* session, ortb200_io_binding** out);
void ortb200_release_io_binding(ortb200_io_binding* binding);
int ortb200_io_binding_bind_input(ortb200_io_binding* binding, const char* name, const ortb200_tensor_view* tensor);
int ortb200_io_binding_bind_output(ortb200_io_binding* binding, const char* name, const ortb200_tensor_view* tensor);
int ortb200_io_binding_bind_output_to_device(ortb200_io_binding* binding, const char* name, int device_type, int device_id);
int ortb200_io_binding_clear_inputs(ortb200_io_binding* binding);
int ortb200_io_binding_clear_outputs(ortb200_io_binding* binding);
int ortb200_io_binding_synchronize_inputs(ortb200_io_binding* binding);
int ortb200_io_binding_synchronize_outputs(ortb200_io_binding* binding);
int ortb200_run_with_binding(ortb200_session* session, const ortb200_run_options* options, ortb200_io_binding* binding);
int ortb200_io_binding_output_count(const ortb200_io_binding* binding, size_t* out);
int ortb200_io_binding_output_name(const ortb200_io_binding* binding, size_t index, const char** out);
/* A new handle on bound output `index` after a run (release with ortb200_release_value). */
int ortb200_io_binding_output_value(ortb200_io_binding* binding, size_t index, ortb200_value** out);

/* A tensor allocated and owned by the runtime (host, pinned host with device_type 2, or CUDA). */
int ortb200_create_tensor(int32_t elem_type, const int64_t* dims, int32_t ndim, int device_type, int device_id, ortb200_value** out);
/* Copies `bytes` bytes between a value and caller memory on the host (a device value is staged through the runtime). */
int ortb200_value_copy_from_host(ortb200_value* value, const void* src, size_t bytes);
int ortb200_value_copy_to_host(ortb200_value* value, void* dst, size_t bytes);
int ortb200_value_byte_size(const ortb200_value* value, size_t* out);

/* Tensors of strings.  ortb200_create_string_tensor copies the NUL-terminated strings (row-major, product(dims) of them).
 * An output of string type answers 1 to ortb200_value_is_string; its elements are read one by one, the returned pointers
 * stay valid for the life of the process.  ortb200_value_tensor on such a value shows the runtime's internal ids.
 * ortb200_run_with_values runs with runtime-owned values as inputs, which is how tensors of strings are fed. */
int ortb200_create_string_tensor(const char* const* strings, const int64_t* dims, int32_t ndim, ortb200_value** out);
int ortb200_value_is_string(const ortb200_value* value, int* out);
int ortb200_value_string_count(const ortb200_value* value, size_t* out);
int ortb200_value_string_element(const ortb200_value* value, size_t index, const char** out, size_t* length);
int ortb200_value_shape(const ortb200_value* value, int64_t* dims /* room for 8 */, int32_t* ndim);
int ortb200_run_with_values(ortb200_session* session, const ortb200_run_options* options, const char* const* input_names,
                            ortb200_value* const* inputs, size_t num_inputs, const char* const* output_names, size_t num_outputs,
                            ortb200_value** outputs);

/* Environment */
int ortb200_available_provider_count(size_t* out);
int ortb200_available_provider_name(size_t index, const char** out);
int ortb200_set_default_logger_severity(int level);
int ortb200_cuda_device_count(int* out);
int ortb200_cuda_memory_info(int device_id, size_t* free_bytes, size_t* total_bytes);

#ifdef __cplusplus
}
#endif
#endif /* ORTB200_C_API_H_ */
