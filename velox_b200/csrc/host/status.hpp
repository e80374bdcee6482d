// Status codes of the host library and the message of the last failure (per thread).
#pragma once
#include <string>

namespace vxh {

enum Status : int {
    OK = 0,
    ERR_ACCOUNTING = -2,       // a page or slot would be lost, held twice or freed twice
    ERR_VALUE = -3,            // an argument that makes no sense
    ERR_OUT_OF_PAGES = -4,     // a request would outgrow its block table
    ERR_REFUSED = -5,          // a request that could never run
    ERR_UNKNOWN_REQUEST = -6,
};

inline std::string& last_error() {
    thread_local std::string message;
    return message;
}
inline int fail(int code, const std::string& message) {
    last_error() = message;
    return code;
}

}  // namespace vxh
