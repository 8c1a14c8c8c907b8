"""A kernel that gave up on a bounded wait is an error of the call that would
have returned its results (the reference reports device failures of a step as
`Forward` / `Synchronize` errors, src/generate/error.rs). The kernels write the
failure into a record in pinned host memory; here that record and the library
are stand-ins, so the host side is tested without a GPU and without making a
wait run out."""
import ctypes

import pytest

from foundry_b200.kernels import ops


class FakeLibraryCall:
    def __init__(self, log, name):
        self.log, self.name = log, name

    def __call__(self, *args):
        self.log.append(self.name)
        return 0


@pytest.fixture
def record(monkeypatch):
    cleared = []
    fake = (ctypes.c_int * 4)()
    monkeypatch.setattr(ops, "_MIRROR", [fake])
    monkeypatch.setattr(ops, "_fn", lambda name: FakeLibraryCall(cleared, name))
    return fake, cleared


def test_no_failure_is_no_error(record):
    fake, cleared = record
    ops.raise_on_device_failure()
    assert cleared == [] and list(fake) == [0, 0, 0, 0]


@pytest.mark.parametrize("kernel, role, words", [
    (1, 1, ("tcgen05 product", "tile loads")),
    (2, 3, ("paired tcgen05 product", "epilogue")),
    (3, 2, ("prompt attention", "matrix instructions")),
    (9, 7, ("kernel 9", "role 7")),
])
def test_a_recorded_failure_raises_once_and_names_the_place(record, kernel, role, words):
    fake, cleared = record
    fake[0], fake[1], fake[2], fake[3] = kernel, role, 41, 5
    with pytest.raises(ops.KernelError) as caught:
        ops.raise_on_device_failure()
    message = str(caught.value)
    assert all(w in message for w in words) and "block 41" in message and "K block 5" in message
    # the record and the device's status words were cleared: the next check passes
    assert list(fake) == [0, 0, 0, 0]
    assert sorted(cleared) == sorted(ops._STATUS_READERS)
    ops.raise_on_device_failure()


def test_a_library_without_the_record_is_tolerated(monkeypatch):
    monkeypatch.setattr(ops, "_MIRROR", [None])
    ops.raise_on_device_failure()


def test_every_ctypes_signature_matches_its_c_declaration():
    """The launchers are called through ctypes with hand-written argument
    lists; a list that is one entry short shows only as a wrong value on the
    GPU. Compared here with the `extern "C"` declarations in the sources."""
    import glob
    import os
    import re
    from foundry_b200.kernels import library
    source = "".join(open(path).read() for path in glob.glob(os.path.join(library.CSRC, "*.cu")))
    for name, signature in ops._SIGNATURES.items():
        found = re.search(r"FB_API int " + name + r"\((.*?)\)\s*\{", source, re.S)
        assert found, f"{name} has no declaration"
        declared = [a for a in found.group(1).split(",") if a.strip()]
        assert len(declared) == len(signature), f"{name}: {len(declared)} declared, {len(signature)} listed"
        for arg, ctype in zip(declared, signature):
            pointer = "*" in arg or "cudaStream_t" in arg
            assert pointer == (ctype is ctypes.c_void_p), f"{name}: {arg.strip()} listed as {ctype}"
