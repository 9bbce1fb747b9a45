// TEST INFRASTRUCTURE.  A fake hwloc (the library is not installed): one package whose cores are the CPUs this
// process may run on, one processing unit each -- the four functions and the object fields that
// src/runtime/local/vectorized/PipelineHWlocInfo.h:18-63 touches.
#pragma once
#include <sched.h>

#include <vector>

typedef enum { HWLOC_OBJ_PACKAGE, HWLOC_OBJ_CORE, HWLOC_OBJ_PU } hwloc_obj_type_t;
struct hwloc_obj {
    hwloc_obj_type_t type;
    unsigned os_index;
    unsigned arity;
    hwloc_obj **children;
};
typedef hwloc_obj *hwloc_obj_t;
struct hwloc_topology {
    std::vector<hwloc_obj> pus, cores;
    std::vector<hwloc_obj *> pu_ptr, core_ptr;
    hwloc_obj package;
};
typedef hwloc_topology *hwloc_topology_t;

inline int hwloc_topology_init(hwloc_topology_t *t) {
    *t = new hwloc_topology();
    return 0;
}
inline int hwloc_topology_load(hwloc_topology_t t) {
    cpu_set_t set;
    CPU_ZERO(&set);
    sched_getaffinity(0, sizeof(set), &set);
    std::vector<unsigned> cpus;
    for (unsigned c = 0; c < CPU_SETSIZE; c++)
        if (CPU_ISSET(c, &set))
            cpus.push_back(c);
    if (cpus.empty())
        cpus.push_back(0);
    const size_t n = cpus.size();
    t->pus.resize(n);
    t->cores.resize(n);
    t->pu_ptr.resize(n);
    t->core_ptr.resize(n);
    for (size_t i = 0; i < n; i++) {
        t->pus[i] = hwloc_obj{HWLOC_OBJ_PU, cpus[i], 0, nullptr};
        t->pu_ptr[i] = &t->pus[i];
    }
    for (size_t i = 0; i < n; i++) {
        t->cores[i] = hwloc_obj{HWLOC_OBJ_CORE, cpus[i], 1, &t->pu_ptr[i]};
        t->core_ptr[i] = &t->cores[i];
    }
    t->package = hwloc_obj{HWLOC_OBJ_PACKAGE, 0, (unsigned)n, t->core_ptr.data()};
    return 0;
}
inline hwloc_obj_t hwloc_get_next_obj_by_type(hwloc_topology_t t, hwloc_obj_type_t type, hwloc_obj_t prev) {
    return (type == HWLOC_OBJ_PACKAGE && prev == nullptr) ? &t->package : nullptr;
}
inline void hwloc_topology_destroy(hwloc_topology_t t) { delete t; }
