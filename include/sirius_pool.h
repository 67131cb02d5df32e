/*
 * sirius_b200 — C ABI of the page pool and allocators behind the training step (the "mpool"
 * contract of the reference, visible through common/cuda_allocator.{h,cc}; the library itself,
 * third_party/mpool, is an empty submodule in the reference tree).
 *
 * One pool of fixed-size physical pages per GPU; a caching allocator for training and a direct
 * allocator for inference map pool pages into their own virtual ranges. srt_pool_empty_cache()
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

int srt_pool_create(const srt_pool_config* cfg, srt_pool** out);       /* CUDAMemPool::Init */
int srt_pool_destroy(srt_pool* p);
/* CUDAMemPool::AllocWithStream / the PoolEntry deleter (cuda_allocator.cc:125-178). Blocks are aligned
 * to 1024 (train) / 512 (infer) bytes. SRT_ERR_NOMEM when neither virtual range nor free pages suffice
 * (after the OOM handler, if any, had a chance to release memory). */
int srt_pool_alloc(srt_pool* p, int kind, size_t nbytes, void** out);
int srt_pool_free(srt_pool* p, int kind, void* ptr);
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

#ifdef __cplusplus
}
#endif
#endif /* SIRIUS_POOL_H_ */
