// Replaying a recorded sequence of launcher calls from C++.
//
// A forward pass is a few launcher calls per layer, issued from Python one by one; for a prompt of a few hundred
// tokens the interpreter's share of that exceeds the device's.  But the layers of a model with equal parts issue
// the SAME calls with the same arguments, except for the pointers to their own weights, cache and state.  So the
// calls of one layer are recorded (launcher index + argument words), and the other layers of the step are run
// by tb_tape_replay: one call from Python per layer, which substitutes the pointers and calls the launchers
// directly.  The reference's whole step is one native call (models/llama/cuda/src/infer.rs:94-147).
//
// Every file that defines launchers ends with TB_TAPE_REGISTER(name) lines; nothing else has to know a
// launcher's signature: the thunk that unpacks the argument words is generated from the function's own type.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <tuple>
#include <utility>

#define TB_TAPE_MAX_ARGS 24

union TapeArg {
    const void* p;
    int i;
    float f;
    long long l;
    unsigned long long u;
};

struct TapeEntry {
    int fn;                 // index from tb_tape_index
    int n_args;             // without the stream
    unsigned ptr_mask;      // bit j set: argument j is a pointer (subject to substitution)
    int reserved;
    TapeArg args[TB_TAPE_MAX_ARGS];
};

// A range of addresses of the recorded layer and what to add to a pointer inside it for the layer being run.
struct TapeMap {
    unsigned long long base, size;
    long long delta;
};

typedef int (*TapeFn)(const TapeArg*, cudaStream_t);
int tb_tape_register(const char* name, TapeFn fn);

template <typename T> struct TapeGet;
template <typename T> struct TapeGet<T*> {
    static T* get(const TapeArg& a) { return (T*)a.p; }
};
template <> struct TapeGet<int> {
    static int get(const TapeArg& a) { return a.i; }
};
template <> struct TapeGet<float> {
    static float get(const TapeArg& a) { return a.f; }
};
template <> struct TapeGet<long long> {
    static long long get(const TapeArg& a) { return a.l; }
};
template <> struct TapeGet<unsigned long long> {
    static unsigned long long get(const TapeArg& a) { return a.u; }
};

template <auto Fn> struct TapeThunk;
template <typename... Args, int (*Fn)(Args...)> struct TapeThunk<Fn> {
    static_assert(sizeof...(Args) >= 1 && sizeof...(Args) - 1 <= TB_TAPE_MAX_ARGS, "a launcher takes its arguments and a stream");
    template <size_t... I> static int go(const TapeArg* a, cudaStream_t s, std::index_sequence<I...>) {
        using Tup = std::tuple<Args...>;
        return Fn(TapeGet<std::tuple_element_t<I, Tup>>::get(a[I])..., s);
    }
    static int call(const TapeArg* a, cudaStream_t s) { return go(a, s, std::make_index_sequence<sizeof...(Args) - 1>{}); }
};

#define TB_TAPE_REGISTER(fn) static const int tb_tape_index_of_##fn = tb_tape_register(#fn, &TapeThunk<&fn>::call);
