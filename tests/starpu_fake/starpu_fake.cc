// One-worker, run-at-insert implementation of the declarations in ./starpu.h.
// TEST INFRASTRUCTURE ONLY: it exists so that the replacement codelets of
// nntile_b200/starpu/ can be driven through the reference's own Codelet / Handle
// classes without StarPU.
#include "starpu.h"

#include <cstdarg>
#include <cstdlib>
#include <cstring>

struct _starpu_data_state
{
    starpu_variable_interface iface;
    bool owned;
};

static void *g_stream = nullptr;
static uint32_t g_last_footprint = 0;
static int g_last_nbuffers = 0;
static int g_tasks_run = 0;

extern "C" int starpu_is_initialized(void)
{
    return 1;
}

extern "C" void starpu_variable_data_register(starpu_data_handle_t *handle, int home_node,
        uintptr_t ptr, size_t size)
{
    auto *h = new _starpu_data_state();
    std::memset(&h->iface, 0, sizeof(h->iface));
    h->owned = home_node < 0;
    h->iface.ptr = h->owned ? 0 : ptr;       // StarPU-owned memory is not modelled
    h->iface.dev_handle = h->iface.ptr;
    h->iface.elemsize = size;
    *handle = h;
}

extern "C" void starpu_data_unregister(starpu_data_handle_t handle)
{
    delete handle;
}

extern "C" void starpu_data_unregister_no_coherency(starpu_data_handle_t handle)
{
    delete handle;
}

extern "C" void starpu_data_unregister_submit(starpu_data_handle_t handle)
{
    delete handle;                            // every task has already run
}

extern "C" void starpu_data_invalidate_submit(starpu_data_handle_t) {}
extern "C" void starpu_data_set_name(starpu_data_handle_t, const char *) {}

extern "C" int starpu_data_acquire(starpu_data_handle_t, enum starpu_data_access_mode)
{
    return 0;
}

extern "C" int starpu_data_acquire_try(starpu_data_handle_t, enum starpu_data_access_mode)
{
    return 0;
}

extern "C" void starpu_data_release(starpu_data_handle_t) {}

extern "C" void *starpu_data_get_local_ptr(starpu_data_handle_t handle)
{
    return reinterpret_cast<void *>(handle->iface.ptr);
}

extern "C" int starpu_task_insert(struct starpu_codelet *cl, ...)
{
    starpu_task task;
    std::memset(&task, 0, sizeof(task));
    task.cl = cl;
    void *buffers[STARPU_NMAXBUFS];
    va_list ap;
    va_start(ap, cl);
    for(;;)
    {
        const int what = va_arg(ap, int);
        if(what == 0)
        {
            break;
        }
        if(what == STARPU_CL_ARGS)
        {
            task.cl_arg = va_arg(ap, void *);
            task.cl_arg_size = va_arg(ap, size_t);
            continue;
        }
        if(what >= STARPU_ACCESS_MODE_MAX || task.nbuffers >= STARPU_NMAXBUFS)
        {
            va_end(ap);
            return -1;                        // not an access mode, or too many buffers
        }
        starpu_data_handle_t h = va_arg(ap, starpu_data_handle_t);
        task.handles[task.nbuffers] = h;
        task.modes[task.nbuffers] = (enum starpu_data_access_mode)what;
        buffers[task.nbuffers] = &h->iface;
        ++task.nbuffers;
    }
    va_end(ap);
    g_last_nbuffers = task.nbuffers;
    g_last_footprint = (cl->model && cl->model->footprint) ? cl->model->footprint(&task) : 0;
    if(!(cl->where & STARPU_CUDA) || !cl->cuda_funcs[0])
    {
        std::free(task.cl_arg);
        return -2;                            // this fake only has a CUDA worker
    }
    cl->cuda_funcs[0](buffers, task.cl_arg);
    ++g_tasks_run;
    std::free(task.cl_arg);                   // STARPU_CL_ARGS: the runtime frees it
    return 0;
}

extern "C" int starpu_worker_get_id(void)
{
    return 0;
}

// any deterministic mixing function will do for a footprint
extern "C" uint32_t starpu_hash_crc32c_be_n(const void *input, size_t n, uint32_t inputcrc)
{
    const unsigned char *p = static_cast<const unsigned char *>(input);
    uint32_t h = inputcrc ^ 0x811C9DC5u;
    for(size_t i = 0; i < n; ++i)
    {
        h = (h ^ p[i])*16777619u;
    }
    return h;
}

extern "C" void starpu_fake_set_stream(void *cuda_stream)
{
    g_stream = cuda_stream;
}

extern "C" uint32_t starpu_fake_last_footprint(void)
{
    return g_last_footprint;
}

extern "C" int starpu_fake_last_nbuffers(void)
{
    return g_last_nbuffers;
}

extern "C" int starpu_fake_tasks_run(void)
{
    return g_tasks_run;
}

extern "C" cudaStream_t starpu_cuda_get_local_stream(void)
{
    return static_cast<cudaStream_t>(g_stream);
}
