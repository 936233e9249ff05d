#pragma once
// Error convention of the drop-in headers: the reference wrappers return void and leave
// through CUDA_CHECK -> exit(EXIT_FAILURE) (reference include/spbitnet/cuda_utils.h:13-21).
// The C-ABI returns a status instead; these headers restore the reference behaviour.
#include <cstdio>
#include <cstdlib>

#include "../spbitnet_b200.h"

#define SPB200_CHECK(call)                                                                 \
    do {                                                                                   \
        const int spb200_status__ = (call);                                                \
        if (spb200_status__ != SPB_OK) {                                                   \
            std::fprintf(stderr, "spbitnet_b200 error %d at %s:%d: %s\n", spb200_status__, \
                         __FILE__, __LINE__, spb_last_error_string());                     \
            std::exit(EXIT_FAILURE);                                                       \
        }                                                                                  \
    } while (0)
