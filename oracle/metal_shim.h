// Minimal C++ stand-ins for the Metal Shading Language names used by the
// reference's scalar decode functions (address-space qualifiers, short integer
// aliases, half, uint2, as_type).  Lets g++ compile those functions, unmodified
// and from where they lie, into oracle/_ref/libref_decode.so.  Test
// infrastructure only.
#pragma once
#include <cstdint>
#include <cstring>
#define device
#define constant static const
#define threadgroup
#define thread
typedef unsigned char uchar;
typedef unsigned short ushort;
typedef unsigned int uint;
typedef unsigned long ulong;
typedef _Float16 half;
struct uint2 {
    uint x, y;
    uint2(uint a, uint b) : x(a), y(b) {}
};
template <class T, class U> inline T as_type(U v) {
    static_assert(sizeof(T) == sizeof(U), "as_type needs equal sizes");
    T t;
    std::memcpy(&t, &v, sizeof(T));
    return t;
}
