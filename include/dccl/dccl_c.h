/**
 * Flat C interface of libdccl.so, for C programs and foreign-function bindings (the Python package
 * loads these symbols with ctypes). No counterpart in the original, whose API is C++ only.
 *
 * Communicators and streams are opaque pointers; data types, operators and results are the integer
 * values of ncclDataType_t, ncclRedOp_t and ncclResult_t in <dccl/dccl.hpp> (0 = success). No call
 * lets a C++ exception escape: a null communicator gives ncclInvalidArgument.
 */
#ifndef DCCL_C_H
#define DCCL_C_H
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* data types (ncclDataType_t) */
enum { DCCL_INT8 = 0, DCCL_UINT8 = 1, DCCL_INT32 = 2, DCCL_UINT32 = 3, DCCL_INT64 = 4, DCCL_UINT64 = 5,
       DCCL_FLOAT16 = 6, DCCL_FLOAT32 = 7, DCCL_FLOAT64 = 8, DCCL_BFLOAT16 = 9 };
/* operators (ncclRedOp_t) */
enum { DCCL_SUM = 0, DCCL_PROD = 1, DCCL_MAX = 2, DCCL_MIN = 3, DCCL_AVG = 4 };

/* life cycle */
int dccl_comm_init(void** comm);                                   /* rank / world from the environment or ./derecho.cfg */
int dccl_get_unique_id(void* id128);                               /* 128-byte token, made on the process that will be rank 0 */
int dccl_comm_init_rank(void** comm, int nranks, const void* id128, int rank);
int dccl_comm_bind_device(void* comm, int device);                 /* collective: set up the device side now */
int dccl_comm_finalize(void* comm);
int dccl_comm_abort(void* comm);
int dccl_comm_shrink(void* comm, void** newcomm);                  /* survivors of a failure form a smaller group */
int dccl_world_size(void* comm);
int dccl_rank(void* comm);
int dccl_last_error(void* comm, int* code, char* msg, size_t len);
const char* dccl_error_string(int result);
int dccl_has_multicast(void* comm);
unsigned long long dccl_launch_count(void* comm);
int dccl_comm_set_param(void* comm, const char* name, int value);
/* counters of a communicator's device side: "launches", "zero_copy_calls", "symmetric_calls" */
unsigned long long dccl_comm_stat(void* comm, const char* name);
/* 1 when [p, p + bytes) lies in symmetric memory of the communicator (dcclMemAlloc or a memory pool it serves) */
int dccl_is_symmetric(void* comm, const void* p, size_t bytes);
int dccl_cuda_device_count(void);
int dccl_barrier(void* comm);                                       /* host-side barrier over the control plane */
int dccl_debug_check(void* comm);                                   /* guard words of the device pool (DCCL_DEBUG_BOUNDS=1) */
int dccl_topology_json(void* comm, char* out, size_t len);         /* GPUs, peer access, NVLink links, multicast */
int dccl_nvml_link_report(const char* nvml_library, char* out, size_t len);   /* NVML only; CUDA builds */

/* memory */
int dccl_register(void* comm, void* buf, size_t size);
int dccl_deregister(void* comm, void* buf);
int dccl_mem_alloc(void* comm, void** ptr, size_t size);
int dccl_mem_free(void* comm, void* ptr);

/* collectives: stream-ordered for device buffers (stream = cudaStream_t), blocking for host buffers (stream ignored) */
int dccl_all_reduce(const void* send, void* recv, size_t count, int dtype, int op, void* comm, void* stream);
int dccl_reduce_scatter(const void* send, void* recv, size_t recvcount, int dtype, int op, void* comm, void* stream);
int dccl_all_gather(const void* send, void* recv, size_t sendcount, int dtype, void* comm, void* stream);
int dccl_broadcast(const void* send, void* recv, size_t count, int dtype, int root, void* comm, void* stream);
int dccl_reduce(const void* send, void* recv, size_t count, int dtype, int op, int root, void* comm, void* stream);
int dccl_send(const void* send, size_t count, int dtype, int peer, void* comm, void* stream);
int dccl_recv(void* recv, size_t count, int dtype, int peer, void* comm, void* stream);
int dccl_all_to_all(const void* send, void* recv, size_t count, int dtype, void* comm, void* stream);
int dccl_all_to_allv(const void* send, const size_t* sendcounts, const size_t* sdispls, void* recv, const size_t* recvcounts,
                     const size_t* rdispls, int dtype, void* comm, void* stream);
int dccl_gather(const void* send, void* recv, size_t count, int dtype, int root, void* comm, void* stream);
int dccl_scatter(const void* send, void* recv, size_t count, int dtype, int root, void* comm, void* stream);
int dccl_group_start(void);
int dccl_group_end(void);
int dccl_set_algorithm(void* comm, const char* collective, const char* name);
const char* dccl_last_algorithm(void* comm, const char* collective);

/* timestamps (.tt files) */
void dccl_timestamp_log(unsigned long long tag, unsigned long long rank, unsigned long long extra);
void dccl_timestamp_flush(const char* filename, int clear);
void dccl_timestamp_clear(void);
unsigned long long dccl_timestamp_size(void);

/* configuration */
void dccl_config_reload(void);
void dccl_config_set(const char* key, const char* value);
int dccl_config_get(const char* key, char* out, size_t len);

/* small helpers */
size_t dccl_size_of_type(int dtype);
int dccl_parse_type(const char* name);
int dccl_parse_op(const char* name);

#ifdef __cplusplus
}
#endif
#endif /* DCCL_C_H */
