"""The C ABI as a surface, checked without a GPU: the header, the ctypes binding, the built library and the
integration notes must name the same functions; the ctypes structures must have the sizes the C compiler gives
the header's; and the argument checks that need no device must answer with error codes."""
import ctypes as C
import os
import re
import subprocess
import tempfile

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "pagoda_sampler.h")


def _declared():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    return re.findall(r"PGS_API\s+[^;(]*?\b(pgs_[a-z0-9_]+)\s*\(", text)


def test_header_binding_library_and_notes_name_the_same_functions():
    from pagoda_b200 import capi
    names = _declared()
    assert len(names) == len(set(names)) and len(names) >= 30
    assert set(names) == set(capi.EXPORTS), set(names) ^ set(capi.EXPORTS)
    lib = capi.load_library()
    for n in names:
        assert hasattr(lib, n), f"{n} is declared but not exported by the library"
    notes = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    missing = [n for n in names if n not in notes]
    assert not missing, f"INTEGRATION.md does not mention {missing}"


def test_ctypes_structures_have_the_sizes_of_the_header():
    from pagoda_b200 import capi
    src = r'''
#include "pagoda_sampler.h"
#include <stdio.h>
#include <stddef.h>
int main(void) {
    printf("%zu %zu %zu %zu %zu %zu\n", sizeof(pgs_batch_desc), sizeof(pgs_tp_desc), sizeof(pgs_tp_out),
           sizeof(pgs_counters), offsetof(pgs_batch_desc, dump_ids), offsetof(pgs_tp_desc, eos_token_id));
    return 0;
}
'''
    with tempfile.TemporaryDirectory() as d:
        open(os.path.join(d, "t.c"), "w").write(src)
        exe = os.path.join(d, "t")
        subprocess.check_call(["gcc", "-std=c11", "-I", os.path.join(ROOT, "include"), os.path.join(d, "t.c"), "-o", exe])
        got = list(map(int, subprocess.run([exe], capture_output=True, text=True, check=True).stdout.split()))
    assert got == [C.sizeof(capi.BatchDesc), C.sizeof(capi.TpDesc), C.sizeof(capi.TpOut), C.sizeof(capi.Counters),
                   capi.BatchDesc.dump_ids.offset, capi.TpDesc.eos_token_id.offset]


def _static_desc(capi, **over):
    d = capi.BatchDesc()
    d.struct_size = C.sizeof(capi.BatchDesc)
    d.rows, d.vocab, d.row_stride = 2, 1024, 1024
    d.logits, d.token, d.status = 0x1000, 0x2000, 0x3000   # never dereferenced: every check below fails first
    for k, v in over.items():
        setattr(d, k, v)
    return d


@pytest.mark.parametrize("over,code,text", [
    (dict(hist_offsets=0x4000), -1, "together"),                 # offsets without ids
    (dict(hist_ids=0x4000), -1, "together"),                     # ids without offsets
    (dict(mask_table=0x4000, mask_state=0x5000), -1, "grammar tables"),
    (dict(vocab=65537, row_stride=65537), -4, "65536"),
    (dict(logits_mem=1), -1, "device memory"),
    (dict(struct_size=8), -1, "descriptor size"),
])
def test_static_entry_point_rejects_bad_descriptors_before_touching_the_device(over, code, text):
    from pagoda_b200 import capi
    lib = capi.load_library()
    d = _static_desc(capi, **over)
    rc = lib.pgs_sample_batch_static(0, C.byref(d), None)
    assert rc == code
    assert text in lib.pgs_static_last_error().decode()
