// Host-only check of nntile_b200/csrc/per_device.hh: "once" means once per
// device ordinal, a failed initialisation is retried, ordinals out of range are
// served without caching.  Returns 0 when every expectation holds.
#include "../nntile_b200/csrc/per_device.hh"

int main()
{
    nb200::PerDeviceOnce once;
    int calls[4] = {0, 0, 0, 0};
    // first use on device 0 and on device 2: each runs its own initialisation
    if(!once.ensure(0, [&]() { ++calls[0]; return true; })) return 1;
    if(!once.ensure(2, [&]() { ++calls[2]; return true; })) return 2;
    // second use on device 0: cached; device 1 was never initialised by the others
    if(!once.ensure(0, [&]() { ++calls[0]; return true; })) return 3;
    if(once.is_done(1)) return 4;
    if(!once.ensure(1, [&]() { ++calls[1]; return true; })) return 5;
    if(calls[0] != 1 || calls[1] != 1 || calls[2] != 1) return 6;
    // a failure is reported and not remembered
    if(once.ensure(3, [&]() { ++calls[3]; return false; })) return 7;
    if(once.is_done(3)) return 8;
    if(!once.ensure(3, [&]() { ++calls[3]; return true; })) return 9;
    if(calls[3] != 2 || !once.is_done(3)) return 10;
    // negative ordinal: refused; beyond the table: runs every time
    int far = 0;
    if(once.ensure(-1, [&]() { return true; })) return 11;
    once.ensure(nb200::PerDeviceOnce::MAX_DEVICES + 5, [&]() { ++far; return true; });
    once.ensure(nb200::PerDeviceOnce::MAX_DEVICES + 5, [&]() { ++far; return true; });
    return far == 2 ? 0 : 12;
}
