// Skilling's Hilbert transform as a finite-state machine.
//
// The operations the transform applies below a level are "invert all lower bits
// of axis 0" and "exchange all lower bits of axis 0 and axis i", i.e. a signed
// permutation of the three axes that is the same for every lower bit.  The
// state is that signed permutation (6 permutations x 8 flip masks = 48 states);
// a level consumes the 3 raw bits of that level, emits 3 bits of the transposed
// (Gray) code and moves to the next state.  Tables for one level (48 x 8) and
// for two levels at once (48 x 64) are evaluated at compile time from the same
// rules as serialization/hilbert.py:156-175.
#pragma once
#include <stdint.h>

namespace ptv3 {
namespace hlut {

struct State {
    int p[3];   // transformed axis i reads raw axis p[i]
    int f[3];   // ... and is inverted when f[i] is set
};

constexpr int perm_id(const int* p)
{
    // 0:(0,1,2) 1:(0,2,1) 2:(1,0,2) 3:(1,2,0) 4:(2,0,1) 5:(2,1,0)
    return p[0] * 2 + (p[1] > p[2] ? 1 : 0);
}
constexpr State decode_state(int s)
{
    State st{};
    const int pid = s >> 3;
    const int first = pid >> 1;
    int rest[2] = {0, 0};
    int k = 0;
    for (int a = 0; a < 3; ++a)
        if (a != first) rest[k++] = a;
    st.p[0] = first;
    st.p[1] = (pid & 1) ? rest[1] : rest[0];
    st.p[2] = (pid & 1) ? rest[0] : rest[1];
    for (int i = 0; i < 3; ++i) st.f[i] = (s >> (2 - i)) & 1;
    return st;
}
constexpr int encode_state(const State& st)
{
    return perm_id(st.p) * 8 + (st.f[0] << 2 | st.f[1] << 1 | st.f[2]);
}
// raw: 3 bits (axis 0 in bit 2).  Returns out3 | next_state << 3.
constexpr int step(int s, int raw)
{
    State st = decode_state(s);
    int b[3] = {0, 0, 0};
    for (int i = 0; i < 3; ++i) b[i] = ((raw >> (2 - st.p[i])) & 1) ^ st.f[i];
    for (int i = 0; i < 3; ++i) {
        if (b[i]) {
            st.f[0] ^= 1;                       // hilbert.py:163-165
        } else if (i != 0) {                    // hilbert.py:168-175
            const int tp = st.p[0], tf = st.f[0];
            st.p[0] = st.p[i];
            st.f[0] = st.f[i];
            st.p[i] = tp;
            st.f[i] = tf;
        }
    }
    return (b[0] << 2 | b[1] << 1 | b[2]) | (encode_state(st) << 3);
}

struct Table1 {
    uint16_t v[48 * 8];
};
struct Table2 {
    uint16_t v[48 * 64];
};
constexpr Table1 make_table1()
{
    Table1 t{};
    for (int s = 0; s < 48; ++s)
        for (int r = 0; r < 8; ++r) t.v[s * 8 + r] = (uint16_t)step(s, r);
    return t;
}
// two levels: raw6 = (upper level's 3 bits) << 3 | lower level's 3 bits.
// Entry: out6 | next_state << 6.
constexpr Table2 make_table2()
{
    Table2 t{};
    for (int s = 0; s < 48; ++s)
        for (int r = 0; r < 64; ++r) {
            const int a = step(s, r >> 3);
            const int b = step(a >> 3, r & 7);
            t.v[s * 64 + r] = (uint16_t)(((a & 7) << 3 | (b & 7)) | ((b >> 3) << 6));
        }
    return t;
}

}  // namespace hlut
}  // namespace ptv3
