"""Recipe for oracle/_ref/: compiles, from the reference's own sources where they lie, the one piece
of the reference that builds stand-alone for this path -- its ExpertProtocolV2 frame validator
(native/src/glmrt_native.cc: read_le16 / read_le32 / read_le64 / validate_protocol_v2_frame,
called on every RDMA frame pair at glmrt_native.cc:2274-2278).

Test infrastructure only: tests pass the frames this repository's codec encodes through the
reference's validator.  Nothing under oracle/ is imported by the product.

    python oracle/build_ref.py [--reference /path/to/reference]

The rest of the reference's native tree needs CMake, CUDA, generated AOT objects and external
libraries and is not built.  The validator sits in an anonymous namespace of a 4,600-line file, so
the recipe cuts the four functions out of that file (by their signatures, not by line numbers),
compiles them between a prologue and an epilogue of its own (status type from the reference's
header, a `fail`/`ok` pair that keeps the message, one extern "C" entry point) in a temporary
directory, and keeps only the shared object: oracle/_ref/libglmrt_ref_pv2.so.  No reference source
is written into the repository.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT_LIB = os.path.join(OUT_DIR, "libglmrt_ref_pv2.so")
DEFAULT_REFERENCE = "/root/reference"

PROLOGUE = r"""
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <string>
#include "glmrt_native.h"
namespace {
thread_local std::string g_message;
glmrt_status_t fail(glmrt_status_t status, const std::string& message) { g_message = message; return status; }
glmrt_status_t ok() { g_message.clear(); return GLMRT_STATUS_OK; }
"""

EPILOGUE = r"""
}  // namespace
extern "C" int glmrt_ref_validate_protocol_v2_frame(const void* frame, size_t frame_bytes, unsigned kind,
                                                    char* message, size_t message_len) {
  const glmrt_status_t st = validate_protocol_v2_frame(frame, frame_bytes, static_cast<uint16_t>(kind),
                                                       kind == 1 ? "request" : "response");
  if (message != nullptr && message_len != 0) {
    std::strncpy(message, g_message.c_str(), message_len - 1);
    message[message_len - 1] = '\0';
  }
  return static_cast<int>(st);
}
"""

BEGIN_MARK = "uint16_t read_le16(const unsigned char* bytes) {"
END_MARK = "glmrt_status_t compute_host_buffer_plan("


def reference_available(reference: str = DEFAULT_REFERENCE) -> bool:
    return os.path.exists(os.path.join(reference, "native", "src", "glmrt_native.cc"))


def build(reference: str = DEFAULT_REFERENCE, force: bool = False) -> str | None:
    """Returns the path of the shared object, or None when the reference tree is not present
    (then a previously built object, if any, is left as it is)."""
    src = os.path.join(reference, "native", "src", "glmrt_native.cc")
    inc = os.path.join(reference, "native", "include")
    if not os.path.exists(src):
        return OUT_LIB if os.path.exists(OUT_LIB) else None
    if not force and os.path.exists(OUT_LIB) and os.path.getmtime(OUT_LIB) >= max(
            os.path.getmtime(src), os.path.getmtime(os.path.abspath(__file__))):
        return OUT_LIB
    text = open(src).read()
    b, e = text.find(BEGIN_MARK), text.find(END_MARK)
    if b < 0 or e < 0 or e <= b or "validate_protocol_v2_frame" not in text[b:e]:
        raise RuntimeError("the frame validator was not found in " + src)
    gxx = shutil.which("g++")
    if gxx is None:
        raise RuntimeError("g++ not found")
    os.makedirs(OUT_DIR, exist_ok=True)
    with tempfile.TemporaryDirectory() as tmp:
        unit = os.path.join(tmp, "pv2_validate_unit.cc")
        with open(unit, "w") as f:
            f.write(PROLOGUE + text[b:e] + EPILOGUE)
        cmd = [gxx, "-std=c++17", "-O1", "-shared", "-fPIC", "-I", inc, unit, "-o", OUT_LIB]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("g++ failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    return OUT_LIB


if __name__ == "__main__":
    ref = DEFAULT_REFERENCE
    if "--reference" in sys.argv:
        ref = sys.argv[sys.argv.index("--reference") + 1]
    print(build(ref, force="--force" in sys.argv))
