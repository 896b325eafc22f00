/* A stand-in for <starpu.h>.  TEST INFRASTRUCTURE ONLY.
 *
 * Declares the part of the StarPU 1.4 C API that the reference's
 * include/nntile/starpu/{codelet,handle}.hh, src/starpu/{codelet,handle}.cc and
 * the two fused-attention codelets use, with the semantics of a single worker
 * that runs every task at once, inside starpu_task_insert (starpu_fake.cc).
 * StarPU itself is installed neither where this repository is built nor where
 * it is tested; this header lets the replacement codelet sources of
 * nntile_b200/starpu/ be compiled against the reference's own headers and be
 * run end to end.  Names, argument orders and constant meanings follow the
 * public StarPU documentation; the numeric values are private to this fake.
 */
#ifndef NNTILE_B200_TEST_STARPU_FAKE_H
#define NNTILE_B200_TEST_STARPU_FAKE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define STARPU_MAXIMPLEMENTATIONS 4
#define STARPU_NMAXBUFS 16                    /* the reference needs 13 */
#define STARPU_NMAXWORKERS 64
#define STARPU_VARIABLE_NBUFFERS (-1)
#define STARPU_MAIN_RAM 0

#define STARPU_NOWHERE ((1ULL) << 0)
#define STARPU_CPU ((1ULL) << 1)
#define STARPU_CUDA ((1ULL) << 3)
#define STARPU_CUDA_ASYNC (1 << 0)

enum starpu_data_access_mode
{
    STARPU_NONE = 0,
    STARPU_R = (1 << 0),
    STARPU_W = (1 << 1),
    STARPU_RW = (STARPU_R | STARPU_W),
    STARPU_SCRATCH = (1 << 2),
    STARPU_REDUX = (1 << 3),
    STARPU_COMMUTE = (1 << 4),
    STARPU_ACCESS_MODE_MAX = (1 << 7)
};
#define STARPU_RW_COMMUTE (STARPU_RW | STARPU_COMMUTE)
/* argument markers of starpu_task_insert, above every access mode */
#define STARPU_CL_ARGS (1 << 16)

struct _starpu_data_state;
typedef struct _starpu_data_state *starpu_data_handle_t;

typedef void (*starpu_cpu_func_t)(void **, void *);
typedef void (*starpu_cuda_func_t)(void **, void *);

struct starpu_task;

enum starpu_perfmodel_type
{
    STARPU_PERFMODEL_INVALID = 0,
    STARPU_HISTORY_BASED = 3
};

struct starpu_perfmodel
{
    enum starpu_perfmodel_type type;
    const char *symbol;
    uint32_t (*footprint)(struct starpu_task *);
};

struct starpu_codelet
{
    uint32_t where;
    starpu_cpu_func_t cpu_funcs[STARPU_MAXIMPLEMENTATIONS];
    starpu_cuda_func_t cuda_funcs[STARPU_MAXIMPLEMENTATIONS];
    char cuda_flags[STARPU_MAXIMPLEMENTATIONS];
    int nbuffers;
    enum starpu_data_access_mode modes[STARPU_NMAXBUFS];
    struct starpu_perfmodel *model;
    const char *name;
};

struct starpu_task
{
    struct starpu_codelet *cl;
    void *cl_arg;
    size_t cl_arg_size;
    int nbuffers;
    starpu_data_handle_t handles[STARPU_NMAXBUFS];
    enum starpu_data_access_mode modes[STARPU_NMAXBUFS];
};

/* what a codelet body finds behind buffers[i] for a variable */
struct starpu_variable_interface
{
    int id;
    uintptr_t ptr;
    uintptr_t dev_handle;
    size_t offset;
    size_t elemsize;
};

int starpu_is_initialized(void);
void starpu_variable_data_register(starpu_data_handle_t *handle, int home_node, uintptr_t ptr,
        size_t size);
void starpu_data_unregister(starpu_data_handle_t handle);
void starpu_data_unregister_no_coherency(starpu_data_handle_t handle);
void starpu_data_unregister_submit(starpu_data_handle_t handle);
void starpu_data_invalidate_submit(starpu_data_handle_t handle);
void starpu_data_set_name(starpu_data_handle_t handle, const char *name);
int starpu_data_acquire(starpu_data_handle_t handle, enum starpu_data_access_mode mode);
int starpu_data_acquire_try(starpu_data_handle_t handle, enum starpu_data_access_mode mode);
void starpu_data_release(starpu_data_handle_t handle);
void *starpu_data_get_local_ptr(starpu_data_handle_t handle);

/* (mode, handle) pairs, then STARPU_CL_ARGS, pointer, size; 0 ends the list */
int starpu_task_insert(struct starpu_codelet *cl, ...);
int starpu_worker_get_id(void);
uint32_t starpu_hash_crc32c_be_n(const void *input, size_t n, uint32_t inputcrc);

/* --- only in this fake: what the test reads back ------------------------- */
/* stream handed out by starpu_cuda_get_local_stream() */
void starpu_fake_set_stream(void *cuda_stream);
/* footprint and number of buffers of the last inserted task */
uint32_t starpu_fake_last_footprint(void);
int starpu_fake_last_nbuffers(void);
int starpu_fake_tasks_run(void);

#ifdef __cplusplus
}
#endif

/* starpu_cuda.h */
#if defined(__cplusplus) && defined(NNTILE_USE_CUDA)
#include <cuda_runtime_api.h>
extern "C" cudaStream_t starpu_cuda_get_local_stream(void);
#endif

#endif /* NNTILE_B200_TEST_STARPU_FAKE_H */
