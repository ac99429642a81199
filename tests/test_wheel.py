"""The wheel of the package: its archive holds the wrapper, the library and the C ABI headers; RECORD's hashes match;
the unpacked tree imports (loading the library needs no GPU) and exports the ABI."""
import base64
import hashlib
import os
import subprocess
import sys
import zipfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_wheel_contents_and_import(tmp_path):
    sys.path.insert(0, ROOT)
    from ozaki_blackwell_b200 import build_wheel
    path = build_wheel.build(str(tmp_path / "dist"), rebuild=False)
    assert os.path.basename(path).endswith("-py3-none-linux_x86_64.whl")
    with zipfile.ZipFile(path) as z:
        names = set(z.namelist())
        for need in ("ozaki_blackwell_b200/__init__.py", "ozaki_blackwell_b200/_lib.py", "ozaki_blackwell_b200/dist.py",
                     "ozaki_blackwell_b200/libozaki_blackwell.so", "ozaki_blackwell_b200/include/ozb.h"):
            assert need in names, need
        record = [n for n in names if n.endswith(".dist-info/RECORD")]
        assert len(record) == 1
        for line in z.read(record[0]).decode().splitlines():
            arc, digest, size = line.rsplit(",", 2)
            if not digest:
                continue
            data = z.read(arc)
            want = base64.urlsafe_b64encode(hashlib.sha256(data).digest()).rstrip(b"=").decode()
            assert digest == "sha256=" + want and int(size) == len(data), arc
        z.extractall(tmp_path / "site")
    code = ("import ozaki_blackwell_b200 as m, os, sys; l = sys.modules['ozaki_blackwell_b200._lib'];"
            "assert os.path.dirname(m.__file__).startswith(os.getcwd());"
            "assert all(hasattr(l.lib, s) for s in l.SYMBOLS); print(l.lib.ozb_version().decode())")
    env = {k: v for k, v in os.environ.items() if k not in ("PYTHONPATH", "OZB_LIBRARY")}
    out = subprocess.run([sys.executable, "-c", code], cwd=tmp_path / "site", env=env, capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    assert out.stdout.strip()
