/*
 * sirius_b200 — C ABI of the page pool and allocators behind the training step (the "mpool"
 * contract of the reference, visible through common/cuda_allocator.{h,cc}; the library itself,
 * third_party/mpool, is an empty submodule in the reference tree).
 *
 * One pool of fixed-size physical pages per GPU; a caching allocator for training and a direct
 * allocator for inference map pool pages into their own virtual ranges; the pool may be private to one
 * process or shared between the server and the trainer processes (srt_pool_create_shared / srt_pool_attach). srt_pool_empty_cache()
 * marks every page that holds no live block FREE: that is the memory handover.
 *
 * Unlike the reference, a page that goes back to the pool stays mapped in the range it leaves (a
 * physical page may be mapped in several ranges at once). When that slot is needed again and its page
 * is still free, the allocator takes it back without a driver call; otherwise it unmaps the slot then
 * and maps another page. A trainer and an inference worker that trade the same pages back and forth
 * therefore reach a steady state with no map/unmap calls on the handover path; on the shared machines
 * this was measured on, single cuMemUnmap calls took between 1 ms and 0.8 s. unmap_on_release = 1
 * restores the reference's behaviour (unmap at empty-cache time).
 */
#ifndef SIRIUS_POOL_H_
#define SIRIUS_POOL_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct srt_pool srt_pool;
enum { SRT_POOL_TRAIN = 0, SRT_POOL_INFER = 1 };              /* MemType::kTrain / kInfer */
enum { SRT_POOL_BACKEND_CUDA_VMM = 0, SRT_POOL_BACKEND_HOST = 1 };

typedef struct srt_pool_config { /* mpool::PagesPoolConf + VMMAllocatorConfig, cuda_allocator.cc:61-99 */
  int device;
  int backend;            /* SRT_POOL_BACKEND_* (HOST: mmap/mprotect stand-in for CPU tests) */
  size_t page_nbytes;     /* 0 = 32 MiB (CUDAMemPool::PageNbytes, cuda_allocator.h:81-87); rounded up to the
                             allocation granularity of the device */
  size_t pool_nbytes;     /* COLTRAIN_SHARED_TENSOR_POOL_GB worth of pages, created up front */
  int train_va_scale;     /* 0 = 8: virtual range of the training allocator in multiples of the pool */
  int infer_va_scale;     /* 0 = 1 */
  int unmap_on_release;   /* 0 = keep the mapping of a released page (see above); 1 = unmap it, as mpool does */
} srt_pool_config;

int srt_pool_create(const srt_pool_config* cfg, srt_pool** out);       /* CUDAMemPool::Init, one process */
/* The pool shared between processes, as the reference's is between the inference server and the trainers
 * (CUDAMemPool::Init builds its pool and allocators as mpool::SharableObject in POSIX shared memory, created by
 * whoever comes first with cleanup and opened by the others, common/cuda_allocator.cc:61-99, segment names
 * common/util.h:113-118). srt_pool_create_shared creates the pages, a segment "/<name>" with the page ownership
 * table, the usage counters of both sides and the process-shared pool lock, and serves the pages' shareable
 * handles (POSIX file descriptors) on the abstract Unix socket "srt_pool.<name>" for as long as the pool
 * lives. srt_pool_attach (any other process, any time; waits up to timeout_ms for the owner) imports the pages
 * and builds its own training and inference allocators over them: virtual addresses are per process, physical
 * pages and their ownership are common, so srt_pool_empty_cache in one process makes pages available to
 * srt_pool_alloc in the other. srt_pool_stat reports both sides from either process. Destroying an attached
 * pool returns the pages that process still held; the owner should be destroyed last. A segment left by a
 * crashed owner is never attached to: attaching goes through the owner's socket, which dies with it. */
int srt_pool_create_shared(const srt_pool_config* cfg, const char* name, srt_pool** out);
int srt_pool_attach(const char* name, int device, int timeout_ms, srt_pool** out);
int srt_pool_destroy(srt_pool* p);
/* CUDAMemPool::AllocWithStream / the PoolEntry deleter (cuda_allocator.cc:125-178). Blocks are aligned
 * to 1024 (train) / 512 (infer) bytes. SRT_ERR_NOMEM when neither virtual range nor free pages suffice
 * (after the OOM handler, if any, had a chance to release memory). */
int srt_pool_alloc(srt_pool* p, int kind, size_t nbytes, void** out);
int srt_pool_free(srt_pool* p, int kind, void* ptr);
/* Gives up the memory of a live block while its owner keeps the address (an intermediate tensor of a killed
 * batch that the framework will free later, torch_allocator_plugin.cc:343-369): the range is not handed out again
 * until srt_pool_free is called on it, but counts as free space for srt_pool_empty_cache. */
int srt_pool_hollow(srt_pool* p, int kind, void* ptr);
/* CUDAMemPool::FreeTrainLocals -> CachingAllocator::EmptyCache (cuda_allocator.cc:304-307). */
int srt_pool_empty_cache(srt_pool* p, int kind, size_t* released_bytes);
enum { SRT_POOL_STAT_INFER_USAGE = 0, SRT_POOL_STAT_TRAIN_USAGE, SRT_POOL_STAT_TRAIN_PEAK, SRT_POOL_STAT_TRAIN_ALL,
       SRT_POOL_STAT_FREE_PAGES, SRT_POOL_STAT_POOL_NBYTES, SRT_POOL_STAT_PAGE_NBYTES, SRT_POOL_STAT_NUM_MAP,
       SRT_POOL_STAT_NUM_UNMAP, SRT_POOL_STAT_INFER_ALLOCATED,
       SRT_POOL_STAT_NUM_REUSE /* slots that took their kept page back without a driver call */ };
int64_t srt_pool_stat(srt_pool* p, int which);                         /* cuda_allocator.cc:259-302 */
/* RegisterOOMHandler (cuda_allocator.cc:311-328): called without the pool lock when an allocation
 * cannot be served; the allocation is retried once afterwards. */
typedef void (*srt_pool_oom_fn)(void* user, int kind, size_t nbytes);
int srt_pool_set_oom_handler(srt_pool* p, srt_pool_oom_fn fn, void* user);

/* ---- the PyTorch allocator seam ----------------------------------------------------------------------
 * The reference replaces PyTorch's CUDA allocator with a C++ subclass whose raw_alloc_with_stream / raw_delete
 * go to the pool's training allocator, whose recordStream keeps a freed block out of circulation until the
 * streams that used it have passed the free, and which can drop all tagged intermediate tensors at once
 * (pytorch/torch_col/csrc/torch_allocator_plugin.cc:36-43 install, :108-178 alloc / free, :200-229 recordStream,
 * :322-375 tagging and ReleaseIntermMemory, :383-412 ProcessEvents; signatures torch_allocator_plugin.h:47-100).
 * srt_alloc / srt_free have the signature torch.cuda.memory.CUDAPluggableAllocator loads by name:
 *
 *   torch.cuda.memory.change_current_allocator(
 *       torch.cuda.memory.CUDAPluggableAllocator("libsirius_b200.so", "srt_alloc", "srt_free"))
 *
 * srt_pool_init makes the process-wide default pool of a device first (CUDAMemPool::Init): it creates a shared
 * pool named <shm prefix>_pool_dev<device> (the prefix of common/util.h:113-132: user and SIRIUS_PORT), or, with
 * COLTRAIN_HAS_SHARED_TENSOR_SERVER=1 and cleanup = 0, attaches to the one the server process created.
 * srt_pool_default hands that pool to the step executors (srt_resnet_create with a pool). srt_alloc returns
 * NULL on failure with the reason in srt_last_error() (it cannot return a status); everything else returns a
 * status and never aborts the process. Any thread may call; one mutex orders the calls, taken before the
 * pool's own lock.
 * srt_tag_model_begin / _end bracket model and optimizer construction (nothing allocated in between is an
 * intermediate); srt_tag_interm marks a live block as a saved-for-backward tensor; srt_release_interm frees all
 * marked blocks while the framework still holds their pointers (a killed batch), returns the pages they leave
 * empty to the pool, and makes the later srt_free of those pointers a no-op. */
int srt_pool_init(int device, size_t nbytes, int cleanup);
int srt_pool_shutdown(int device);
int srt_pool_default(int device, srt_pool** out);
void* srt_alloc(size_t nbytes, int device, void* stream);
void srt_free(void* ptr, size_t nbytes, int device, void* stream);
int srt_record_stream(void* ptr, int device, void* stream);
int srt_empty_cache(int device, size_t* released_bytes);
int srt_tag_model_begin(void);
int srt_tag_model_end(void);
int srt_tag_interm(void* ptr, int device);
int srt_untag_interm(int device);
int srt_release_interm(int device, size_t* released_bytes);
int64_t srt_pool_stat_dev(int device, int which);                      /* srt_pool_stat of the default pool */
/* Counters of the seam: calls served, frees that had to wait for a recorded stream, blocks still waiting, live blocks. */
int srt_alloc_counters(int device, int64_t* allocs, int64_t* frees, int64_t* deferred, int64_t* pending, int64_t* live);

#ifdef __cplusplus
}
#endif
#endif /* SIRIUS_POOL_H_ */
