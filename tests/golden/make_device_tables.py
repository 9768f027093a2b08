"""Produce ``device_tables.npz`` (needs a B200): compiles and runs ``device_tables.cu`` beside this
file and stores its two lookup tables.  See ``oracle/nvfp4.py`` ("device" mode) for their use."""
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


def main(out_dir: Path):
    with tempfile.TemporaryDirectory() as tmp:
        exe, raw = Path(tmp) / "device_tables", Path(tmp) / "device_tables.bin"
        subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17",
                        str(HERE / "device_tables.cu"), "-o", str(exe)], check=True)
        subprocess.run([str(exe), str(raw)], check=True)
        buf = raw.read_bytes()
    sf = np.frombuffer(buf[:32768], dtype=np.uint8)
    inv = np.frombuffer(buf[32768:32768 + 512], dtype=np.float32)
    out_dir.mkdir(parents=True, exist_ok=True)
    np.savez_compressed(out_dir / "device_tables.npz", sf_of_absmax=sf, inv_of_sf=inv)
    print("wrote", out_dir / "device_tables.npz")


if __name__ == "__main__":
    main(Path(sys.argv[1]) if len(sys.argv) > 1 else HERE)
