// The table of launchers that can be replayed, and the replay itself (see tape.h).
#include "tape.h"

#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"

namespace {
struct Slot {
    std::string name;
    TapeFn fn;
};
std::vector<Slot>& table() {
    static std::vector<Slot> t;      // built while the library is loaded, by the files' static initialisers
    return t;
}
std::mutex& table_lock() {
    static std::mutex m;
    return m;
}
}  // namespace

int tb_tape_register(const char* name, TapeFn fn) {
    std::lock_guard<std::mutex> hold(table_lock());
    table().push_back({name, fn});
    return (int)table().size() - 1;
}

extern "C" {
// Index of a launcher for TapeEntry.fn, or -1 if it did not register.
int tb_tape_index(const char* name) {
    std::lock_guard<std::mutex> hold(table_lock());
    for (size_t i = 0; i < table().size(); ++i)
        if (table()[i].name == name) return (int)i;
    return -1;
}

// Run the n recorded calls in order on stream s.  A pointer argument that lies inside [base, base + size) of a map
// is moved by that map's delta (first match).  Returns 0, or the first launcher's error with its position in
// *failed_at; a launcher that refuses its sizes (TB_ERR_UNSUPPORTED) is an error here: the recorded call did run.
int tb_tape_replay(const TapeEntry* entries, int n, const TapeMap* maps, int n_maps, int* failed_at, cudaStream_t s) {
    const int known = (int)table().size();
    for (int e = 0; e < n; ++e) {
        const TapeEntry& t = entries[e];
        if (t.fn < 0 || t.fn >= known || t.n_args < 0 || t.n_args > TB_TAPE_MAX_ARGS) {
            if (failed_at) *failed_at = e;
            return TB_ERR_ARG;
        }
        TapeArg a[TB_TAPE_MAX_ARGS];
        std::memcpy(a, t.args, sizeof(TapeArg) * t.n_args);
        for (int j = 0; j < t.n_args; ++j) {
            if (!(t.ptr_mask >> j & 1u) || !a[j].p) continue;
            const unsigned long long p = (unsigned long long)a[j].p;
            for (int m = 0; m < n_maps; ++m)
                if (p >= maps[m].base && p - maps[m].base < maps[m].size) {
                    a[j].p = (const void*)(p + (unsigned long long)maps[m].delta);
                    break;
                }
        }
        const int rc = table()[t.fn].fn(a, s);
        if (rc != 0) {
            if (failed_at) *failed_at = e;
            return rc;
        }
    }
    return 0;
}
}
