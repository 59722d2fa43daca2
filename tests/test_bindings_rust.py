"""The Rust declarations a datago maintainer would link against (bindings/rust/datago-b200-sys) name exactly the entry
points the header declares and the library exports.  No Rust toolchain exists in the build container, so the crate is
checked as text: every `DG_API` function of include/datago_b200.h must appear as a `pub fn` and vice versa."""
import os
import re

import datago_b200

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_rust_declarations_match_the_header_and_the_library():
    header = open(os.path.join(ROOT, "include", "datago_b200.h")).read()
    rust = open(os.path.join(ROOT, "bindings", "rust", "datago-b200-sys", "src", "lib.rs")).read()
    in_header = set(re.findall(r"DG_API\s+[\w\s\*]+?\b(dg_\w+)\s*\(", header))
    in_rust = set(re.findall(r"pub fn (dg_\w+)\s*\(", rust))
    assert in_header == in_rust, (sorted(in_header - in_rust), sorted(in_rust - in_header))
    assert in_header == set(datago_b200.EXPORTS), sorted(in_header ^ set(datago_b200.EXPORTS))
    lib = datago_b200.lib()
    assert all(hasattr(lib, name) for name in in_header)
