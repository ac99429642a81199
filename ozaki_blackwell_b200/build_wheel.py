"""Build a binary wheel of this package for B200: `python -m ozaki_blackwell_b200.build_wheel [--out DIR]`.

The wheel carries the Python wrapper and libozaki_blackwell.so (sm_100a machine code only, CUDA runtime linked
statically, so that the NVIDIA driver is its only dependency at run time). The role is that of the reference's
python/build.sh + python/make_wheel.py, which pack a multi-architecture build of its library the same way; here the
library is built by csrc/Makefile and the archive is written directly (a wheel is a zip with three metadata files),
so that no build backend has to be installed.
"""
import argparse
import base64
import hashlib
import os
import subprocess
import zipfile

HERE = os.path.dirname(os.path.abspath(__file__))
NAME = "ozaki_blackwell_b200"
PY_FILES = ("__init__.py", "__main__.py", "_lib.py", "dist.py", "gemm_bench.py", "exact_f8_bench.py")
LIB = "libozaki_blackwell.so"


def _version():
    with open(os.path.join(HERE, "__init__.py")) as f:
        for line in f:
            if line.startswith("__version__"):
                return line.split('"')[1]
    raise RuntimeError("no __version__ in __init__.py")


def _record_line(arcname, data):
    digest = base64.urlsafe_b64encode(hashlib.sha256(data).digest()).rstrip(b"=").decode()
    return f"{arcname},sha256={digest},{len(data)}"


def build(out_dir, rebuild=True):
    if rebuild:
        subprocess.run(["make", "-s", "-C", os.path.join(HERE, "csrc")], check=True)
    if not os.path.exists(os.path.join(HERE, LIB)):
        raise FileNotFoundError(f"{LIB} is not built")
    version = _version()
    tag = "py3-none-linux_x86_64"
    info = f"{NAME}-{version}.dist-info"
    headers = [("include/ozb.h", os.path.join(HERE, "..", "include", "ozb.h")),
               ("include/ozaki2.hpp", os.path.join(HERE, "..", "include", "ozaki2.hpp"))]
    files = [(f"{NAME}/{f}", os.path.join(HERE, f)) for f in PY_FILES + (LIB,)]
    files += [(f"{NAME}/{arc}", path) for arc, path in headers if os.path.exists(path)]   # the C ABI travels with the library
    metadata = "\n".join([
        "Metadata-Version: 2.1", f"Name: {NAME.replace('_', '-')}", f"Version: {version}",
        "Summary: FP64-accurate GEMM from INT8 tensor-core products (Ozaki scheme II) for NVIDIA B200 (sm_100a)",
        "Requires-Python: >=3.9", "Requires-Dist: numpy", ""])
    wheel = "\n".join(["Wheel-Version: 1.0", "Generator: ozaki_blackwell_b200.build_wheel", "Root-Is-Purelib: false", f"Tag: {tag}", ""])
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, f"{NAME}-{version}-{tag}.whl")
    record = []
    with zipfile.ZipFile(path, "w", zipfile.ZIP_DEFLATED) as z:
        for arc, src in files:
            with open(src, "rb") as f:
                data = f.read()
            z.writestr(arc, data)
            record.append(_record_line(arc, data))
        for arc, text in ((f"{info}/METADATA", metadata), (f"{info}/WHEEL", wheel)):
            z.writestr(arc, text)
            record.append(_record_line(arc, text.encode()))
        record.append(f"{info}/RECORD,,")
        z.writestr(f"{info}/RECORD", "\n".join(record) + "\n")
    return path


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--out", default=os.path.join(HERE, "..", "dist"))
    ap.add_argument("--no-rebuild", action="store_true", help="pack the library as it is")
    a = ap.parse_args()
    print(build(a.out, not a.no_rebuild))
