// Error reporting and version of the C ABI.
#include "common.cuh"

namespace bpt {

char *error_buffer() {
    static thread_local char buf[512] = {0};
    return buf;
}

int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

}  // namespace bpt

extern "C" const char *bpt_last_error(void) { return bpt::error_buffer(); }
extern "C" int bpt_version(void) { return 1; }
