/*
 * C-ABI of the B200 vendor runtime (libdipu_vendor_b200.so).
 *
 * DIPU's vendor contract is a set of C++ free functions in namespace dipu::devapis whose
 * signatures leak torch types (c10::DeviceIndex, at::ScalarType, c10d::ReduceOp).  This header
 * is the same contract with plain C types; csrc/vendor/torch_abi/{deviceimpl.cpp,
 * communicatorimpl.cpp} are the thin C++ wrappers with the exact reference signatures.
 * Each group cites the reference declaration it stands for, as
 *   dipu/torch_dipu/csrc_dipu/runtime/device/<file>:<lines>   (path inside the reference project).
 *
 * Error convention: every function returns b200Status_t; on failure b200_last_error() holds a
 * thread-local message (the C++ wrappers turn it into the c10::Error DIPU expects).  Sticky CUDA
 * errors are cleared where the reference clears them (malloc with ERR_NOMEM, event query).
 * Thread safety: all functions may be called from any thread; nothing relies on a per-process
 * current device except where the reference does (the *current* device is whatever
 * b200_set_device last set on the calling thread, as in CUDA).
 */
#ifndef DIPU_B200_VENDOR_C_API_H_
#define DIPU_B200_VENDOR_C_API_H_

#include <stddef.h>
#include <stdint.h>
#include <sys/types.h>

#include "dipu_b200/peer_space.h"

#ifdef __cplusplus
extern "C" {
#endif

#define B200_API __attribute__((visibility("default")))

typedef enum {
    B200_SUCCESS = 0,     /* devapis::OpStatus::SUCCESS      basedef.h:55-59 */
    B200_ERR_UNKNOWN = 1, /* devapis::OpStatus::ERR_UNKNOWN */
    B200_ERR_NOMEM = 2,   /* devapis::OpStatus::ERR_NOMEM   */
    B200_ERR_TIMEOUT = 3, /* a bounded device-side wait gave up (no reference counterpart) */
} b200Status_t;

typedef enum { /* devapis::EventStatus  basedef.h:53 */
    B200_EVENT_PENDING = 0,
    B200_EVENT_RUNNING = 1,
    B200_EVENT_DEFERRED = 2,
    B200_EVENT_READY = 3,
} b200EventStatus_t;

typedef void* b200Stream_t; /* cudaStream_t   vendor/cuda/vendorapi.h:44 */
typedef void* b200Event_t;  /* cudaEvent_t    vendor/cuda/vendorapi.h:46 */
typedef struct b200Comm* b200Comm_t; /* stands for diclComm_t = ncclComm_t  vendorapi.h:48 */

#define B200_UNIQUE_ID_BYTES 128 /* DICL_UNIQUE_ID_BYTES_SIZE = NCCL_UNIQUE_ID_BYTES  vendor/cuda/communiatorimpl.cpp:66 */
typedef struct { char internal[B200_UNIQUE_ID_BYTES]; } b200UniqueId; /* commUniqueId: trivially copyable, sent through the c10d store */

typedef struct { /* devapis::DIPUDeviceProperties  basedef.h:80-86 */
    char name[256];
    size_t total_global_mem;
    int32_t major;
    int32_t minor;
    int32_t multi_processor_count;
} b200DeviceProperties;

B200_API const char* b200_last_error(void);

/* ---- device: deviceapis.h:23-46 ------------------------------------------------------------- */
B200_API b200Status_t b200_initialize_vendor(void);
B200_API b200Status_t b200_finalize_vendor(void);
B200_API b200Status_t b200_current_device(int* device);
B200_API b200Status_t b200_get_device_properties(int device, b200DeviceProperties* props);
B200_API b200Status_t b200_get_device_status(int device, size_t* free_bytes, size_t* total_bytes);
B200_API b200Status_t b200_set_device(int device);
B200_API b200Status_t b200_reset_device(int device);
B200_API b200Status_t b200_sync_device(void);
B200_API b200Status_t b200_check_last_error(void);
B200_API b200Status_t b200_get_device_count(int* count);
B200_API b200Status_t b200_get_driver_version(int* version);
B200_API b200Status_t b200_get_runtime_version(int* version);

/* ---- streams: deviceapis.h:48-64 -------------------------------------------------------------- */
B200_API b200Status_t b200_create_stream(b200Stream_t* stream, int high_priority);
B200_API b200Status_t b200_destroy_stream(b200Stream_t stream);
B200_API b200Status_t b200_destroy_stream_on(b200Stream_t stream, int device);
B200_API b200Status_t b200_release_stream(void);
B200_API b200Status_t b200_sync_stream(b200Stream_t stream);
B200_API int b200_stream_not_null(b200Stream_t stream);
B200_API b200Status_t b200_stream_wait_event(b200Stream_t stream, b200Event_t event);
B200_API int b200_is_stream_empty(b200Stream_t stream);

/* ---- events: deviceapis.h:70-82 ---------------------------------------------------------------- */
B200_API b200Status_t b200_create_event(b200Event_t* event); /* timing on unless DIPU_CUDA_EVENT_TIMING=0 */
B200_API b200Status_t b200_destroy_event(b200Event_t event);
B200_API b200Status_t b200_wait_event(b200Event_t event);
B200_API b200Status_t b200_record_event(b200Event_t event, b200Stream_t stream);
B200_API b200Status_t b200_event_elapsed_time(float* ms, b200Event_t start, b200Event_t end);
B200_API b200Status_t b200_get_event_status(b200Event_t event, b200EventStatus_t* status);

/* ---- memory: deviceapis.h:87-124 ----------------------------------------------------------------- */
B200_API b200Status_t b200_malloc_host(void** p, size_t nbytes);
B200_API b200Status_t b200_free_host(void* p);
/* returns B200_ERR_NOMEM (error state cleared) when out of memory: the caching allocator then frees its cache and retries */
B200_API b200Status_t b200_malloc_device(void** p, size_t nbytes);
B200_API b200Status_t b200_free_device(void* p);
B200_API int b200_is_pinned_ptr(const void* p);
B200_API b200Status_t b200_memset_async(b200Stream_t stream, void* ptr, int value, size_t nbytes);
B200_API b200Status_t b200_memcpy_d2d(size_t nbytes, int dst_device, void* dst, int src_device, const void* src);
B200_API b200Status_t b200_memcpy_h2d(size_t nbytes, void* dst, const void* src);
B200_API b200Status_t b200_memcpy_d2h(size_t nbytes, void* dst, const void* src);
B200_API b200Status_t b200_memcpy_d2d_async(b200Stream_t stream, size_t nbytes, int dst_device, void* dst, int src_device, const void* src);
B200_API b200Status_t b200_memcpy_h2d_async(b200Stream_t stream, size_t nbytes, void* dst, const void* src);
B200_API b200Status_t b200_memcpy_d2h_async(b200Stream_t stream, size_t nbytes, void* dst, const void* src);

/* ---- caching device allocator ------------------------------------------------------------------------
 * Stands for dipu::getAllocator(DIPU) with DIPU_DEVICE_MEMCACHING_ALGORITHM=TORCH
 * (runtime/core/allocator/DIPUCachingDeviceAllocator.cpp:584-880,1958-2036): per-stream pools of split /
 * coalesced blocks, record_stream with event-deferred reuse, OOM -> free cache -> retry. */
typedef struct { /* the six headline counters of DeviceStats (DIPUCachingDeviceAllocator.h:44-98) + retries */
    int64_t allocated_bytes, allocated_bytes_peak;
    int64_t reserved_bytes, reserved_bytes_peak;
    int64_t active_blocks, segments;
    int64_t num_alloc_retries, num_ooms;
    int64_t num_device_mallocs, num_cache_hits;
} b200AllocStats;

B200_API b200Status_t b200_cache_alloc(void** p, size_t nbytes, int device, b200Stream_t stream);
B200_API b200Status_t b200_cache_free(void* p);
B200_API b200Status_t b200_cache_record_stream(void* p, b200Stream_t stream);
B200_API b200Status_t b200_cache_empty(void); /* empty_cache(): return every unused segment to the driver */
B200_API b200Status_t b200_cache_stats(int device, b200AllocStats* stats);
B200_API b200Status_t b200_cache_reset_peak(int device);
/* "key:value,key:value" as in DIPU_TORCH_ALLOCATOR_CONF (DIPUCachingDeviceAllocator.cpp:454-496):
 * max_split_size_mb, expandable_segments:True|False (one growing segment per pool and stream, see b200_expandable_*),
 * garbage_collection_threshold (accepted, unused), roundup_power2_divisions (accepted, unused) */
B200_API b200Status_t b200_cache_configure(const char* conf);
/* Test backend: replaces cudaMalloc/cudaFree/events by host-side fakes with `capacity` bytes of pretend HBM, so the
 * allocator's policy (split, merge, retry ladder, deferred frees) is testable without a GPU. capacity 0 restores CUDA.
 * pending_events != 0 makes every recorded event stay "not ready" until b200_cache_fake_complete_events(). */
B200_API b200Status_t b200_cache_use_fake_backend(size_t capacity, int pending_events);
B200_API b200Status_t b200_cache_fake_complete_events(void);

/* Allocation hooks with the signatures torch.cuda.memory.CUDAPluggableAllocator expects, so that a stock torch build can
 * use this allocator for every device tensor, as DIPU does through c10::SetAllocator
 * (runtime/core/allocator/DIPUCachingAllocator.cpp:336-342). */
B200_API void* b200_torch_alloc(ssize_t size, int device, void* stream);
B200_API void b200_torch_free(void* ptr, ssize_t size, int device, void* stream);

/* ---- caching pinned-host allocator (runtime/core/allocator/DIPUCachingHostAllocator.cpp:99-299) --------- */
B200_API b200Status_t b200_host_cache_alloc(void** p, size_t nbytes);
B200_API b200Status_t b200_host_cache_free(void* p);
B200_API b200Status_t b200_host_cache_record_stream(void* p, b200Stream_t stream);
B200_API b200Status_t b200_host_cache_empty(void);

/* ---- expandable segments ------------------------------------------------------------------------------------
 * The vendor side of DIPU's ExpandableSegment (runtime/core/allocator/ExpandableSegment.h:105-136: map, unmap, addPeer,
 * ptr, size; factory vendorCreateExpandableSegment(device, stream, size, peers), CUDA implementation
 * vendor/cuda/CUDAExpandableSegment.cpp:15-187). A segment reserves virtual addresses for 9/8 of the device's memory;
 * map() backs the pages a range touches with physical memory and returns the mapped range, or an empty range when the
 * device is out of memory; unmap() releases the whole pages inside a range after waiting for the segment's stream.
 * page_size: a multiple of 2 MiB (DIPU uses 2 MiB for its small pool, 20 MiB for the large one). */
B200_API b200Status_t b200_expandable_create(void** segment, int device, b200Stream_t stream, size_t page_size, const int* peers, int npeers);
B200_API b200Status_t b200_expandable_destroy(void* segment);
B200_API b200Status_t b200_expandable_map(void* segment, void* ptr, size_t size, void** mapped_ptr, size_t* mapped_size);
B200_API b200Status_t b200_expandable_unmap(void* segment, void* ptr, size_t size, void** unmapped_ptr, size_t* unmapped_size);
B200_API b200Status_t b200_expandable_add_peer(void* segment, int device);
B200_API void* b200_expandable_ptr(void* segment);
B200_API size_t b200_expandable_size(void* segment);
B200_API size_t b200_expandable_mapped_bytes(void* segment);

/* ---- stream / event pools --------------------------------------------------------------------------------
 * runtime/core/DIPUStream.cpp:38-131 (one lazily created default stream + 8 round-robin pool streams per
 * device) and runtime/core/DIPUEventPool.cpp:11-100 (events recycled per device, never destroyed before exit). */
B200_API b200Status_t b200_default_stream(int device, b200Stream_t* stream);
B200_API b200Status_t b200_stream_from_pool(int device, b200Stream_t* stream);
B200_API b200Status_t b200_event_from_pool(b200Event_t* event);
B200_API b200Status_t b200_event_to_pool(b200Event_t event);
B200_API b200Status_t b200_release_all_pools(void);

/* ---- stream capture into CUDA graphs ---------------------------------------------------------------------------------
 * No counterpart in the reference (DIPU replays the eager op stream from the host every step). A latency-bound step such as
 * single-token decode is captured once - every DIOPI call, copy and collective enqueued on `stream` between begin and end,
 * including work forked to other streams through events - and replayed with one launch, which removes the per-op host cost.
 * Nothing that synchronises or allocates through the driver may run while capturing: warm the step up first. */
typedef struct CUgraphExec_st* b200GraphExec_t;
B200_API b200Status_t b200_graph_begin_capture(b200Stream_t stream);
B200_API b200Status_t b200_graph_end_capture(b200Stream_t stream, b200GraphExec_t* exec);
B200_API b200Status_t b200_graph_launch(b200GraphExec_t exec, b200Stream_t stream);
B200_API b200Status_t b200_graph_destroy(b200GraphExec_t exec);

/* ---- DICL communicator: diclapis.h:20-82 ------------------------------------------------------------------
 * dtype: a diopiDtype_t value (include/diopi/diopirt.h); bool travels as uint8 like the reference's NCCL map
 * (vendor/cuda/communiatorimpl.cpp:44-52). op: b200ReduceOp_t, same order as c10d::ReduceOp (communiatorimpl.cpp:35-41). */
typedef enum { B200_REDUCE_SUM = 0, B200_REDUCE_AVG = 1, B200_REDUCE_PRODUCT = 2, B200_REDUCE_MIN = 3, B200_REDUCE_MAX = 4 } b200ReduceOp_t;

B200_API int b200_dicl_unique_id_bytes(void);
B200_API b200Status_t b200_dicl_get_unique_id(b200UniqueId* id);
B200_API b200Status_t b200_dicl_comm_init_rank(b200Comm_t* comm, int nranks, const b200UniqueId* id, int rank, int local_device);
B200_API b200Status_t b200_dicl_comm_destroy(b200Comm_t comm);
/* B200_SUCCESS when the communicator is healthy, B200_ERR_UNKNOWN when an asynchronous error is pending
 * (the reference returns the opposite by mistake, communiatorimpl.cpp:68-76) */
B200_API b200Status_t b200_dicl_get_comm_async_error(b200Comm_t comm);
B200_API b200Status_t b200_dicl_all_reduce(const void* send, void* recv, size_t count, int dtype, int op, b200Comm_t comm, b200Stream_t stream);
B200_API b200Status_t b200_dicl_broadcast(const void* send, void* recv, size_t count, int dtype, int root, b200Comm_t comm, b200Stream_t stream);
B200_API b200Status_t b200_dicl_all_gather(const void* send, void* recv, size_t send_count, int dtype, b200Comm_t comm, b200Stream_t stream);
B200_API b200Status_t b200_dicl_reduce(const void* send, void* recv, size_t count, int dtype, int op, int root, b200Comm_t comm, b200Stream_t stream);
B200_API b200Status_t b200_dicl_reduce_scatter(const void* send, void* recv, size_t recv_count, int dtype, int op, b200Comm_t comm, b200Stream_t stream);
B200_API b200Status_t b200_dicl_send(const void* send, size_t count, int dtype, int peer, b200Comm_t comm, b200Stream_t stream);
B200_API b200Status_t b200_dicl_recv(void* recv, size_t count, int dtype, int peer, b200Comm_t comm, b200Stream_t stream);
/* weak (absent) in the reference's CUDA vendor, diclapis.h:62-82; here: grouped send/recv */
B200_API b200Status_t b200_dicl_all_to_all_equal_split(const void* send, void* recv, size_t count, int dtype, b200Comm_t comm, b200Stream_t stream);
B200_API b200Status_t b200_dicl_all_to_all_unequal_split(const void* send, const size_t* send_counts, const size_t* send_displs, void* recv,
                                                         const size_t* recv_counts, const size_t* recv_displs, int dtype, b200Comm_t comm,
                                                         b200Stream_t stream);
B200_API b200Status_t b200_dicl_get_comm_name(char* name, size_t capacity, b200Comm_t comm);
B200_API b200Status_t b200_dicl_comm_rank(b200Comm_t comm, int* rank, int* nranks);

/* All-reduce (SUM) of small messages in ONE kernel over peer memory (CUDA IPC mappings of every rank's staging buffer,
 * NVLink loads / stores, bounded flag waits) instead of a library collective: for the latency-bound partial sums of
 * tensor-parallel decode, which the reference sends through diclAllReduce = ncclAllReduce
 * (runtime/distributed/ProcessGroupDICL.cpp:539-567, vendor/cuda/communiatorimpl.cpp:84-92). No reference counterpart.
 * create is collective over `comm` (handles are exchanged with the communicator's all-gather); every rank must call
 * all_reduce with the same count, in the same order; float16 / bfloat16 / float32, buffers 16-byte aligned, byte count a
 * multiple of 16 and at most max_bytes; in place (send == recv) is allowed. The sum is formed in fp32 in rank order, so
 * every rank gets bit-identical results. status: 0, or 1 once a wait for a peer ran into its limit (1 s by default).
 * destroy is collective too: each rank drains its device and meets the others in a one-element all-reduce before its
 * blocks are unmapped and freed (a peer may still be reading this rank's staging when this rank's own kernel has ended).
 * set_wait_limit_ns: limit of every flag wait in the peer-memory kernels this process launches afterwards (all-reduce and
 * reduce-gather); 0 restores the default of one second. reset_status clears a reported time-out. */
B200_API b200Status_t b200_dicl_peer_reduce_create(void** handle, b200Comm_t comm, size_t max_bytes, b200Stream_t stream);
B200_API b200Status_t b200_dicl_peer_all_reduce(void* handle, const void* send, void* recv, size_t count, int dtype, b200Stream_t stream);
B200_API int b200_dicl_peer_reduce_status(void* handle);
B200_API b200Status_t b200_dicl_peer_reduce_reset_status(void* handle);
B200_API b200Status_t b200_dicl_peer_reduce_destroy(void* handle);
B200_API void b200_dicl_peer_set_wait_limit_ns(unsigned long long ns);

/* Peer space: staging slots, result slots and flags every rank of a communicator allocates and maps from all peers
 * (layout: dipu_b200/peer_space.h), for a row-parallel linear whose all-reduce is fused into the compute kernels: the
 * matrix product pushes its tiles to the owners of their rows (diopiB200MmPush, include/diopi/functions_b200.h), and
 * peer_reduce_gather then forms residual + sum of the partial products for the rows this rank owns and writes them into
 * result slot `slot` of EVERY rank. The reference does this as mm followed by ProcessGroupDICL::allreduce
 * (runtime/distributed/ProcessGroupDICL.cpp:539-567) and an aten add. No reference counterpart.
 *   create            collective over `comm`; slot_bytes a multiple of 16384; the largest [rows, cols] result must fit a slot.
 *   create_emulated   a group of `nranks` inside one process on the current device (tests): handles[r] is rank r's view.
 *                     Launch the products of all ranks first, then the reductions with final_wait = 0, all on one stream.
 *   describe          geometry and this process's mappings, by value, for diopiB200MmPush.
 *   result            device address of result slot `slot` on this rank: [rows, cols] dense. It keeps its content until a
 *                     later reduce_gather call on the same slot starts on ANY rank, so re-use a slot only after every reader
 *                     of its old content has been ordered before this rank's next product on that slot.
 *   reduce_gather     every rank, same order, same (slot, epoch, rows, cols); epoch as passed to the products. float16 (8)
 *                     or bfloat16 (12); residual [rows, cols] dense, 16-byte aligned, or NULL (only the owned rows are read).
 *                     All calls on one handle must be enqueued on one stream. final_wait = 1 except under emulation.
 *   status            0, or 1 once a wait for a peer ran into its limit (1 s by default). A CTA whose wait ran out does not
 *                     announce completion, so the peers' final waits run out as well: every rank reports the failure.
 *   check             B200_SUCCESS, or B200_ERR_TIMEOUT with a message once status is non-zero (DICL_ERR_UNDEF one level up).
 *   reset_status      clears a reported time-out; the next calls on the space work as before. */
B200_API b200Status_t b200_dicl_peer_space_create(void** handle, b200Comm_t comm, size_t slot_bytes, int slots, b200Stream_t stream);
B200_API b200Status_t b200_dicl_peer_space_create_emulated(void** handles, int nranks, size_t slot_bytes, int slots);
B200_API b200Status_t b200_dicl_peer_space_describe(void* handle, b200PeerSpace* out);
B200_API void* b200_dicl_peer_space_result(void* handle, int slot);
B200_API b200Status_t b200_dicl_peer_reduce_gather(void* handle, int slot, uint32_t epoch, const void* residual, int64_t rows, int64_t cols,
                                                   int dtype, int final_wait, b200Stream_t stream);
B200_API int b200_dicl_peer_space_status(void* handle);
B200_API b200Status_t b200_dicl_peer_space_check(void* handle);
B200_API b200Status_t b200_dicl_peer_space_reset_status(void* handle);
B200_API b200Status_t b200_dicl_peer_space_destroy(void* handle);

#ifdef __cplusplus
}
#endif
#endif /* DIPU_B200_VENDOR_C_API_H_ */
