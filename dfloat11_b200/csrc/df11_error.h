// Per-thread error message behind df11_last_error().
#pragma once

// Stores a printf-style message for the calling thread and returns `code`.
int df11_fail(int code, const char *fmt, ...)
#if defined(__GNUC__)
    __attribute__((format(printf, 2, 3)))
#endif
    ;
