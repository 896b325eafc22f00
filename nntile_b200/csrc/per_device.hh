// Once-per-device bookkeeping for state that CUDA keeps per (process, device):
// kernel attributes such as the dynamic shared-memory opt-in, symbol addresses,
// helper streams.  One process may drive several GPUs (one task-runtime worker
// thread per device, as the reference's StarPU CUDA workers do), so "done once"
// must mean "done once on THIS device".
//
// Plain C++ (no CUDA headers): the device ordinal is an argument, which also
// lets a host-only test drive the bookkeeping without a GPU.
#pragma once

#include <atomic>

namespace nb200 {

class PerDeviceOnce
{
public:
    static constexpr int MAX_DEVICES = 64;

    // Runs `init()` (returning true on success) unless it already succeeded for
    // `device`.  A failure is not remembered: the next call tries again.  Two
    // threads racing on the same device may both run `init`, which must
    // therefore be idempotent (every use here is).  Ordinals outside
    // [0, MAX_DEVICES) are served without caching.
    template<typename Init>
    bool ensure(int device, Init &&init)
    {
        if(device < 0)
        {
            return false;
        }
        if(device >= MAX_DEVICES)
        {
            return init();
        }
        if(done_[device].load(std::memory_order_acquire) != 0)
        {
            return true;
        }
        if(!init())
        {
            return false;
        }
        done_[device].store(1, std::memory_order_release);
        return true;
    }

    bool is_done(int device) const
    {
        return device >= 0 && device < MAX_DEVICES
                && done_[device].load(std::memory_order_acquire) != 0;
    }

private:
    std::atomic<unsigned char> done_[MAX_DEVICES] = {};
};

} // namespace nb200
