// Mapping from device-side status words to the library's return code: a word that is
// non-zero means some bounded device-side wait of the call gave up, so the call's
// results are not to be trusted.  Plain host code (no CUDA), so that the rule is
// testable on a machine without a GPU.
#pragma once
#include "b200p.h"

namespace b200p {

inline int status_words_rc(const int* words, int n) {
    for (int i = 0; i < n; ++i)
        if (words[i] != 0) return B200P_E_TIMEOUT;
    return B200P_OK;
}

} // namespace b200p
