"""TEST INFRASTRUCTURE: builds the CPU checker libraries.

  oracle/_build/libkcg_oracle.so   from oracle/host_matmul.c (always)
  oracle/_ref/libkcg_ref.so        the reference's own hostMatmul (matmul.cpp), compiled from
                                   the reference tree where it lies, only when that tree exists.
                                   The function body is extracted into oracle/_ref/ (git-ignored)
                                   at build time; it is never stored in this repository.

Both are compiled with -O2 -ffp-contract=off so that the restatement and the reference agree bit
for bit. The rest of the reference's CPU-side code (main(), the HIP kernels in the same file)
needs the HIP runtime headers and is not buildable here.
"""
import os
import re
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
def reference_dir() -> str:
    """Where the reference's source tree lies: $KCG_REFERENCE_DIR, else a directory named `reference`
    beside this repository. It may not exist (a GPU box has none)."""
    return os.environ.get("KCG_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


REFERENCE_DIR = reference_dir()
CFLAGS = ["-O2", "-ffp-contract=off", "-fPIC", "-shared"]


def build_port() -> str:
    out_dir = os.path.join(HERE, "_build")
    os.makedirs(out_dir, exist_ok=True)
    out = os.path.join(out_dir, "libkcg_oracle.so")
    src = os.path.join(HERE, "host_matmul.c")
    if not os.path.exists(out) or os.path.getmtime(out) < os.path.getmtime(src):
        subprocess.check_call(["gcc", *CFLAGS, "-o", out, src])
    return out


def extract_host_matmul(text: str) -> str:
    """The `template <typename T> void hostMatmul(...) {...}` definition, by brace matching."""
    m = re.search(r"template\s*<\s*typename\s+T\s*>\s*void\s+hostMatmul\s*\(", text)
    if not m:
        raise RuntimeError("hostMatmul not found in the reference's matmul.cpp")
    i = text.index("{", m.end())
    depth, j = 0, i
    while True:
        if text[j] == "{":
            depth += 1
        elif text[j] == "}":
            depth -= 1
            if depth == 0:
                break
        j += 1
    return text[m.start():j + 1] + "\n"


def build_ref():
    """Returns the path of libkcg_ref.so, or None when the reference tree is absent."""
    src = os.path.join(REFERENCE_DIR, "matmul.cpp")
    out_dir = os.path.join(HERE, "_ref")
    out = os.path.join(out_dir, "libkcg_ref.so")
    if not os.path.exists(src):
        return out if os.path.exists(out) else None
    os.makedirs(out_dir, exist_ok=True)
    with open(src, encoding="utf-8", errors="replace") as f:
        body = extract_host_matmul(f.read())
    with open(os.path.join(out_dir, "hostMatmul_extract.inc"), "w") as f:
        f.write(body)
    subprocess.check_call(["g++", *CFLAGS, "-I", HERE, "-o", out, os.path.join(HERE, "ref_wrapper.cpp")])
    return out


if __name__ == "__main__":
    print(build_port())
    print(build_ref())
    sys.exit(0)
