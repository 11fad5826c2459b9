"""List the plugin's parameters: name, environment variable, present value, where the value came
from and what it does.

    python -m aws_ofi_nccl_b200.utils.params              # table
    python -m aws_ofi_nccl_b200.utils.params --markdown   # the table of docs/PARAMETERS.md
    python -m aws_ofi_nccl_b200.utils.params --json

Every parameter NAME is read from ``B200NET_NAME`` or, for scripts written for the reference
plugin, ``OFI_NCCL_NAME`` (reference: include/nccl_ofi_param.h). The list comes from the built
library itself (``b200net_describe_parameters``), so it cannot drift from the code.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import sys
from pathlib import Path

LIB = Path(__file__).resolve().parent.parent / "lib" / "libnccl-net-ofi-b200.so"


def describe(lib_path: Path = LIB) -> list[dict]:
    lib = C.CDLL(str(lib_path))
    fn = lib.b200net_describe_parameters
    fn.restype = C.c_size_t
    fn.argtypes = [C.c_char_p, C.c_size_t]
    need = fn(None, 0)
    buf = C.create_string_buffer(need + 1)
    fn(buf, need + 1)
    return json.loads(buf.value.decode())


def markdown(rows: list[dict]) -> str:
    out = ["| parameter (`B200NET_…` / `OFI_NCCL_…`) | default | description |", "|---|---|---|"]
    for r in rows:
        doc = r["doc"].replace("|", "\\|")
        out.append(f"| `{r['name']}` | `{r['value'] or ' '}` | {doc} |")
    return "\n".join(out)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--markdown", action="store_true")
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--lib", default=str(LIB))
    args = ap.parse_args(argv)
    rows = describe(Path(args.lib))
    if args.json:
        print(json.dumps(rows, indent=1))
    elif args.markdown:
        print(markdown(rows))
    else:
        width = max(len(r["name"]) for r in rows)
        for r in rows:
            print(f"{r['name']:<{width}}  {r['value']!s:<12}  [{r['source']}]  {r['doc']}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
