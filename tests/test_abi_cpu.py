"""The C ABI without a GPU: the shared object loads, exports every function the header declares, the ctypes
structures have the C layout, and argument validation answers before any CUDA work."""
import ctypes as C
import os
import re
import subprocess
import tempfile

from lithos_metal_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "lithos_b200.h")


def declared_functions():
    text = open(HEADER).read()
    return re.findall(r"^LM_API\s+[\w\s\*]+?\b(lm_\w+)\s*\(", text, flags=re.M)


def test_library_exports_every_declared_symbol():
    L = _lib.lib()
    names = declared_functions()
    assert set(names) == set(_lib.EXPORTS) and len(names) >= 10
    for n in names:
        assert getattr(L, n) is not None
    assert L.lm_abi_version() == _lib.ABI_VERSION == 3
    assert L.lm_error_string(0) == b"ok" and L.lm_error_string(-2).startswith(b"workspace")


def test_ctypes_structs_match_the_c_layout():
    src = '#include <stdio.h>\n#include "lithos_b200.h"\nint main(){printf("%zu %zu %zu %zu %zu %zu %zu ", sizeof(lm_sample_args), sizeof(lm_verify_args),' \
          ' offsetof(lm_sample_args, out_tokens), offsetof(lm_verify_args, workspace), sizeof(lm_draft_q_args), offsetof(lm_draft_q_args, out_mass),' \
          ' offsetof(lm_verify_args, draft_mass));printf("%zu ", offsetof(lm_verify_args, commit));printf("%zu %zu\\n", sizeof(lm_confidence_args), offsetof(lm_confidence_args, stream));return 0;}\n'
    with tempfile.TemporaryDirectory() as d:
        open(os.path.join(d, "t.c"), "w").write(src)
        subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), "-o", os.path.join(d, "t"), os.path.join(d, "t.c")], check=True)
        out = subprocess.run([os.path.join(d, "t")], capture_output=True, text=True, check=True).stdout.split()
    assert [int(x) for x in out] == [C.sizeof(_lib.SampleArgs), C.sizeof(_lib.VerifyArgs), _lib.SampleArgs.out_tokens.offset,
                                     _lib.VerifyArgs.workspace.offset, C.sizeof(_lib.DraftQArgs), _lib.DraftQArgs.out_mass.offset,
                                     _lib.VerifyArgs.draft_mass.offset, _lib.VerifyArgs.commit.offset, C.sizeof(_lib.ConfidenceArgs), _lib.ConfidenceArgs.stream.offset]


def test_argument_validation_needs_no_device():
    L = _lib.lib()
    a = _lib.SampleArgs()
    assert L.lm_sample(C.byref(a)) == -1                       # struct_size not set
    a.struct_size = C.sizeof(_lib.SampleArgs)
    a.rows, a.vocab = 0, 100
    assert L.lm_sample(C.byref(a)) == 0                        # nothing to do
    a.rows = 4
    assert L.lm_sample(C.byref(a)) == -1                       # null logits
    a.dtype = 7
    assert L.lm_sample(C.byref(a)) == -1
    v = _lib.VerifyArgs()
    v.struct_size = C.sizeof(_lib.VerifyArgs)
    v.n_draft = 0
    assert L.lm_verify(C.byref(v)) == -1
    d = _lib.DraftQArgs()
    assert L.lm_draft_q(C.byref(d)) == -1                      # struct_size not set
    d.struct_size = C.sizeof(_lib.DraftQArgs)
    d.rows, d.vocab, d.temperature = 17, 100, 1.0
    assert L.lm_draft_q(C.byref(d)) == -1                      # more rows than a round has
    c = _lib.ConfidenceArgs()
    c.struct_size = C.sizeof(_lib.ConfidenceArgs)
    c.gamma, c.hidden = 17, 8
    assert L.lm_confidence(C.byref(c)) == -1                   # more positions than a round has
    c.gamma = 0
    assert L.lm_confidence(C.byref(c)) == 0                    # nothing to do
    assert L.lm_argmax(None, 0, 0, 10, 10, None, None, 0, None) == 0
    assert L.lm_argmax(None, 0, 2, 10, 10, None, None, 0, None) == -1
    assert L.lm_workspace_bytes(256, 151936) >= 256 * 16 and L.lm_verify_workspace_bytes(7, 151936) > 0
    # pieces of a vocabulary shard: as many as the merge takes with the other GPUs' (64 records of up to 128 candidates per row), none for
    # large records or short shards; for many rows only as many as keep the records to gather small (or as the shard's length needs)
    assert [L.lm_vocab_pieces(s, 120, 262144 // s, 1) for s in (2, 4, 8)] == [32, 16, 8]
    assert [L.lm_vocab_pieces(s, 104, 262144 // s, 64) for s in (2, 4, 8)] == [8, 4, 2]
    assert L.lm_vocab_pieces(8, 568, 32768, 1) == 1 and L.lm_vocab_pieces(4, 120, 2048, 1) == 1 and L.lm_vocab_pieces(3, 72, 100000, 1) == 16


def test_host_hash_equals_the_oracle():
    import oracle
    L = _lib.lib()
    for args in [(0, 0, 0, 0), (12345, 7, 3001, 0), (2**63 + 5, 1, 4000, 151935)]:
        assert L.lm_uniform01(*args) == oracle.uniform01(*args)
