"""Builds `oracle/_ref/`: the reference itself, as far as this hot path needs it, so that the
parity tests can run the reference's own loader beside this package on a machine that has
no checkout of it (test infrastructure; nothing under `linnet_b200/` imports or runs it).

    python -m oracle.build_ref [path-to-reference-checkout]

What it makes (all of it is git-ignored; nothing of the reference is committed):

* `oracle/_ref/bin/linnet` -- the reference's compiler, compiled from the sources where
  they lie in the checkout with plain `g++ -std=c++23` (every `src/**/*.cpp` except the
  plan-runner library in `src/runtime`, plus the two headers its CMake files generate from
  templates: the version string and the embedded `stdlib/prelude.linnet`).  The reference's
  own build system is not run.  `linnet.torch.load` calls this binary to plan a model and to
  emit its PyTorch source.
* `oracle/_ref/python/linnet`, `oracle/_ref/stdlib`, `oracle/_ref/examples/01-llama` --
  verbatim copies of the reference's Python package, standard library and Llama example
  card, the equivalent of installing its wheel next to this repository.

`environment()` gives the variables a process needs to use them (`LINNET_BIN`, `LINNET_STD`,
`LINNET_HOME`, `PYTHONPATH`); `available()` says whether `oracle/_ref` is complete.
"""

from __future__ import annotations

import os
import re
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
STAMP = OUT / "built-from.txt"


def default_checkout() -> Path:
    """`$LINNET_REFERENCE`, else a directory `reference` beside this repository."""
    env = os.environ.get("LINNET_REFERENCE")
    return Path(env) if env else HERE.parent.parent / "reference"


def available() -> bool:
    return (OUT / "bin" / "linnet").is_file() and (OUT / "python" / "linnet" / "torch" / "__init__.py").is_file() \
        and (OUT / "stdlib" / "quant.linnet").is_file()


def environment(home: Path | str) -> dict[str, str]:
    """Environment of a process that runs the reference out of `oracle/_ref`; `home` is a
    writable directory for the compiler's output cache."""
    env = dict(os.environ)
    env["LINNET_BIN"] = str(OUT / "bin" / "linnet")
    env["LINNET_STD"] = str(OUT / "stdlib")
    env["LINNET_HOME"] = str(home)
    env["PYTHONPATH"] = os.pathsep.join([str(OUT / "python"), str(HERE.parent), env.get("PYTHONPATH", "")]).rstrip(os.pathsep)
    return env


def _version(checkout: Path) -> str:
    text = (checkout / "CMakeLists.txt").read_text(encoding="utf-8")
    found = re.search(r"project\(linnet VERSION ([0-9.]+)", text)
    return found.group(1) if found else "0.0.0"


def _generate_headers(checkout: Path, include: Path) -> None:
    target = include / "linnet"
    target.mkdir(parents=True, exist_ok=True)
    version = (checkout / "cmake" / "version.hpp.in").read_text(encoding="utf-8")
    (target / "version.hpp").write_text(version.replace("@PROJECT_VERSION@", _version(checkout)), encoding="utf-8")
    prelude = (checkout / "cmake" / "prelude.hpp.in").read_text(encoding="utf-8")
    source = (checkout / "stdlib" / "prelude.linnet").read_text(encoding="utf-8")
    (target / "prelude.hpp").write_text(prelude.replace("@LINNET_PRELUDE@", source), encoding="utf-8")


def _stamp_of(checkout: Path) -> str:
    newest = max(p.stat().st_mtime for p in (checkout / "src").rglob("*.cpp"))
    return f"{checkout}\n{newest}\n"


def build(checkout: Path | None = None, force: bool = False, jobs: int | None = None) -> Path:
    checkout = Path(checkout) if checkout is not None else default_checkout()
    if not (checkout / "src" / "cli" / "main.cpp").is_file():
        raise FileNotFoundError(f"no reference checkout at {checkout}")
    if not force and available() and STAMP.is_file() and STAMP.read_text() == _stamp_of(checkout):
        return OUT
    OUT.mkdir(exist_ok=True)
    objects = OUT / "obj"
    objects.mkdir(exist_ok=True)
    generated = OUT / "generated"
    _generate_headers(checkout, generated)

    sources = sorted(p for p in (checkout / "src").rglob("*.cpp") if "runtime" not in p.relative_to(checkout).parts)
    flags = ["-std=c++23", "-O1", "-w", "-I", str(checkout / "include"), "-I", str(generated)]

    def compile_one(source: Path) -> Path:
        obj = objects / ("_".join(source.relative_to(checkout / "src").with_suffix("").parts) + ".o")
        if force or not obj.exists() or obj.stat().st_mtime < source.stat().st_mtime:
            done = subprocess.run(["g++", *flags, "-c", str(source), "-o", str(obj)], capture_output=True, text=True)
            if done.returncode != 0:
                raise RuntimeError(f"g++ failed on {source}:\n{done.stderr[-4000:]}")
        return obj

    with ThreadPoolExecutor(max_workers=jobs or os.cpu_count() or 4) as pool:
        built = list(pool.map(compile_one, sources))
    (OUT / "bin").mkdir(exist_ok=True)
    link = subprocess.run(["g++", "-o", str(OUT / "bin" / "linnet"), *map(str, built)], capture_output=True, text=True)
    if link.returncode != 0:
        raise RuntimeError(f"linking the reference compiler failed:\n{link.stderr[-4000:]}")

    for relative, target in (("python/linnet/src/linnet", "python/linnet"), ("stdlib", "stdlib"),
                             ("examples/01-llama", "examples/01-llama")):
        destination = OUT / target
        if destination.exists():
            for path in [destination, *destination.rglob("*")]:
                if path.is_dir():
                    path.chmod(0o755)
            shutil.rmtree(destination)
        shutil.copytree(checkout / relative, destination, ignore=shutil.ignore_patterns("__pycache__"),
                        copy_function=shutil.copyfile)
        for path in [destination, *destination.rglob("*")]:  # a read-only checkout copies read-only
            path.chmod(path.stat().st_mode | 0o200 | (0o100 if path.is_dir() else 0))
    shutil.rmtree(objects)  # only the linked binary travels
    STAMP.write_text(_stamp_of(checkout))
    return OUT


if __name__ == "__main__":
    where = build(Path(sys.argv[1]) if len(sys.argv) > 1 and not sys.argv[1].startswith("-") else None,
                  force="--force" in sys.argv)
    print(where)
