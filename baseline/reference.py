"""The unmodified reference (phcool/Layer_Quant) beside this library: vendoring recipe and loader.

    python baseline/reference.py --from /path/to/Layer_Quant      # copies into baseline/_ref/

``baseline/_ref/`` is git-ignored: the reference's files never enter this repository's history, they
only travel with a working copy to the machine that runs the benchmark.  The recipe copies the
reference's ``hybrid_quant/`` package and its ``run_nemotron_8b_decode_degradation.py`` byte for
byte and writes their SHA-256 digests to ``baseline/_ref/MANIFEST.json``; nothing is edited.

``load()`` imports the two hot-path modules of that copy under private module names, so they never
collide with this repository's own ``hybrid_quant`` aliases, and returns them.  They are real Triton
code: importing them needs Triton and running them needs a GPU.  Users: the ``triton_ref_*`` cells of
``bench.py`` (the reference's kernels timed on the same GPU as this library's) and the GPU parity
tests that feed both implementations the same inputs.
"""
from __future__ import annotations

import argparse
import hashlib
import importlib.util
import json
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_DIR = HERE / "_ref"
COPIED = ("hybrid_quant", "run_nemotron_8b_decode_degradation.py")


def _digest(path: Path) -> str:
    return hashlib.sha256(path.read_bytes()).hexdigest()


def vendor(src: Path, dst: Path = REF_DIR) -> dict:
    """Copy the reference's hot-path package and driver script from ``src`` to ``dst`` unmodified."""
    src = Path(src).resolve()
    if not (src / "hybrid_quant" / "int4_8b_attention.py").exists():
        raise FileNotFoundError(f"{src} is not a Layer_Quant checkout (hybrid_quant/int4_8b_attention.py missing)")
    if dst.exists():
        shutil.rmtree(dst)
    dst.mkdir(parents=True)
    manifest = {}
    for name in COPIED:
        s = src / name
        if s.is_dir():
            for f in sorted(s.rglob("*.py")):
                rel = f.relative_to(src)
                (dst / rel).parent.mkdir(parents=True, exist_ok=True)
                shutil.copyfile(f, dst / rel)
                manifest[str(rel)] = _digest(f)
        else:
            shutil.copyfile(s, dst / name)
            manifest[name] = _digest(s)
    (dst / "MANIFEST.json").write_text(json.dumps({"source": "phcool/Layer_Quant", "files": manifest}, indent=1) + "\n")
    return manifest


def available() -> bool:
    return (REF_DIR / "hybrid_quant" / "int4_8b_attention.py").exists()


def verify() -> None:
    """Raise if a vendored file no longer matches the digest recorded when it was copied."""
    manifest = json.loads((REF_DIR / "MANIFEST.json").read_text())["files"]
    for rel, digest in manifest.items():
        if _digest(REF_DIR / rel) != digest:
            raise RuntimeError(f"baseline/_ref/{rel} differs from the copy the recipe made; re-run baseline/reference.py")


def _load_file(name: str, path: Path):
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod  # triton.jit reads the source through the module's file
    spec.loader.exec_module(mod)
    return mod


def load():
    """(int4_8b_attention, mamba_state_8b_kernel) of the vendored reference, unmodified."""
    if not available():
        raise RuntimeError("baseline/_ref is empty: run `python baseline/reference.py --from <Layer_Quant checkout>` first")
    verify()
    ia = _load_file("layer_quant_reference_int4_8b_attention", REF_DIR / "hybrid_quant" / "int4_8b_attention.py")
    mk = _load_file("layer_quant_reference_mamba_state_8b_kernel", REF_DIR / "hybrid_quant" / "mamba_state_8b_kernel.py")
    return ia, mk


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--from", dest="src", required=True, help="path of a phcool/Layer_Quant checkout")
    args = ap.parse_args()
    manifest = vendor(Path(args.src))
    print(f"copied {len(manifest)} files into {REF_DIR}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
