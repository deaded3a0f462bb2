#include "registry.h"

#include <map>
#include <tuple>

namespace tfft {

typedef std::tuple<int, int, int, int, int> Key;

static std::map<Key, KernelEntry>& table() {
    static std::map<Key, KernelEntry> t;  // function-local: safe during static registration
    return t;
}

void register_kernel(int dtype, int role, int logm, int loge, int logc, int ft, const void* fn, int threads,
                     size_t smem, int remlast) {
    KernelEntry& e = table()[Key(dtype, role, logm, loge, logc)];
    e.fn[ft] = fn;
    e.threads = threads;
    e.remlast = remlast;
    if (ft == 3) e.smem_csum = smem;
    else e.smem = smem;
}

const KernelEntry* find_kernel(int dtype, int role, int logm, int loge, int logc) {
    auto it = table().find(Key(dtype, role, logm, loge, logc));
    return it == table().end() ? nullptr : &it->second;
}

int registered_kernel_count() {
    int n = 0;
    for (auto& kv : table())
        for (int f = 0; f < 4; ++f) n += kv.second.fn[f] != nullptr;
    return n;
}

}  // namespace tfft
