"""The Rust shim is source only (no Rust toolchain in the image).  What can be checked without one: the generated
`extern "C"` block names exactly the entry points the headers declare, it is up to date with the headers, and every
`sys::nrs_*` call in the hand-written modules names a declared entry point and passes the declared number of
arguments."""
import re
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
SHIM = ROOT / "rust_shim"


def _declared():
    from neuralrs_b200 import _lib
    return _lib.declared_functions()


def test_sys_rs_declares_exactly_the_header_symbols():
    text = (SHIM / "src" / "cuda" / "sys.rs").read_text()
    in_rust = set(re.findall(r"pub fn (nrs_\w+)\(", text))
    assert in_rust == set(_declared())


def test_sys_rs_is_up_to_date_with_the_headers():
    sys.path.insert(0, str(SHIM))
    import gen_sys
    assert gen_sys.generate() == (SHIM / "src" / "cuda" / "sys.rs").read_text(), "run python rust_shim/gen_sys.py"


def _calls(text):
    """(name, argument count) of every sys::nrs_*(...) call, by bracket matching."""
    out = []
    for m in re.finditer(r"sys::(nrs_\w+)\(", text):
        depth, i, args, cur = 1, m.end(), 0, ""
        while depth:
            ch = text[i]
            if ch in "([{":
                depth += 1
            elif ch in ")]}":
                depth -= 1
            if depth == 1 and ch == ",":
                args += 1
                cur = ""
            elif depth:
                cur += ch
            i += 1
        out.append((m.group(1), args + (1 if cur.strip() else 0)))
    return out


def test_hand_written_modules_call_declared_entry_points_with_the_right_arity():
    decl = _declared()
    seen = set()
    for f in sorted((SHIM / "src" / "cuda").glob("*.rs")):
        if f.name == "sys.rs":
            continue
        types = {"nrs_ctx", "nrs_node", "nrs_adamw", "nrs_trainer", "nrs_dp", "nrs_checkpoint", "nrs_layer_spec", "nrs_named_tensor",
                 "nrs_poll_fn"}
        for name in re.findall(r"sys::(nrs_\w+)\b", f.read_text()):      # also entry points passed as function pointers
            if name in types:
                continue
            assert name in decl, f"{f.name}: {name} is not declared in include/*.h"
            seen.add(name)
        for name, nargs in _calls(f.read_text()):
            assert name in decl, f"{f.name}: {name} is not declared in include/*.h"
            assert nargs == len(decl[name][1]), f"{f.name}: {name} called with {nargs} arguments, declared with {len(decl[name][1])}"
            seen.add(name)
    # the operator surface of the reference's GPU path is covered
    for needed in ("nrs_op_conv2d", "nrs_op_matmul", "nrs_op_maxpool2d", "nrs_op_layernorm", "nrs_cross_entropy",
                   "nrs_cross_entropy_backward", "nrs_adamw_step_nodes", "nrs_to_cuda", "nrs_zero_grad", "nrs_node_backward",
                   "nrs_op_transformer_block", "nrs_op_mha", "nrs_op_embedding", "nrs_bucket_register", "nrs_backward_graph_dp"):
        assert needed in seen, needed
