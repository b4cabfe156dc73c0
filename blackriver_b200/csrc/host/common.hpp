// Error handling and small utilities shared by the host side.
//
// The reference terminates the process on any failed check (blackriver/common.hpp:15-81).
// Here br_panic / br_assert throw br::Panic instead: left uncaught (as in train_bloom) the
// process still dies with the same message, while the C API for embedding hosts can catch it
// and hand back an error string.
#pragma once

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace br {

struct Panic : public std::runtime_error {
    using std::runtime_error::runtime_error;
};

[[noreturn]] inline void panic_at(const char* file, int line, const std::string& msg) {
    std::ostringstream ss;
    ss << "**Panic:\t" << msg << "\nSource:\t\t" << file << ", line " << line;
    std::cerr << ss.str() << std::endl;
    throw Panic(ss.str());
}

inline void assert_at(bool ok, const char* expr, const char* file, int line, const std::string& msg) {
    if (!ok) {
        std::ostringstream ss;
        ss << "**Assert failed:\t" << msg << "\nExpected:\t" << expr << "\nSource:\t\t" << file << ", line " << line;
        std::cerr << ss.str() << std::endl;
        throw Panic(ss.str());
    }
}

// Reads a raw little-endian file of T.  The reference reads in 1024-element blocks and
// requires the element count to be a multiple of 1024 (blackriver/common.hpp:83-101); any
// length that is a whole number of elements is accepted here.
template <typename T>
inline void read_data(const char* fileName, std::vector<T>& out) {
    std::ifstream in(fileName, std::ios::binary | std::ios::ate);
    if (!in) panic_at(__FILE__, __LINE__, std::string("can't open ") + fileName);
    std::streamsize bytes = in.tellg();
    in.seekg(0, std::ios::beg);
    if (bytes < 0 || bytes % (std::streamsize)sizeof(T) != 0) panic_at(__FILE__, __LINE__, std::string("bad file length: ") + fileName);
    out.resize((size_t)bytes / sizeof(T));
    if (bytes > 0 && !in.read(reinterpret_cast<char*>(out.data()), bytes)) panic_at(__FILE__, __LINE__, std::string("short read: ") + fileName);
}

}  // namespace br

#define br_panic(Msg) ::br::panic_at(__FILE__, __LINE__, (Msg))
#define br_assert(Expr, Msg) ::br::assert_at(static_cast<bool>(Expr), #Expr, __FILE__, __LINE__, (Msg))

// A failed operator is fatal at the facade, as in the reference (blackriver/common.hpp:59-63).
#define op_check(ret, Msg)                                                         \
    do {                                                                           \
        if ((ret) != ::br::OP_OK) {                                                \
            ::br::panic_at(__FILE__, __LINE__, std::string(Msg) + " returned " + std::to_string((int)(ret))); \
        }                                                                          \
        return (ret);                                                              \
    } while (0)

#define BR_CUDA_CHECK(call)                                                                              \
    do {                                                                                                 \
        cudaError_t s_ = (call);                                                                         \
        if (s_ != cudaSuccess) ::br::panic_at(__FILE__, __LINE__, std::string(#call) + ": " + cudaGetErrorString(s_)); \
    } while (0)

#define BR_NCCL_CHECK(call)                                                                              \
    do {                                                                                                 \
        ncclResult_t s_ = (call);                                                                        \
        if (s_ != ncclSuccess) ::br::panic_at(__FILE__, __LINE__, std::string(#call) + ": " + ncclGetErrorString(s_)); \
    } while (0)
