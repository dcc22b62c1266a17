"""The C ABI: the library loads without a GPU, exports every symbol the header declares, and its
argument validation answers without touching a device."""
import ctypes
import re
from pathlib import Path

import b200norm

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "b200norm.h"


def declared_functions():
    text = HEADER.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b2n_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for required in ("b2n_layer_norm_fwd", "b2n_layer_norm_bwd", "b2n_rms_norm_fwd", "b2n_rms_norm_bwd",
                     "b2n_softmax_fwd", "b2n_softmax_bwd", "b2n_nll_loss_fwd", "b2n_nll_loss_bwd", "b2n_cross_entropy_bwd",
                     "b2n_masked_softmax_fwd", "b2n_masked_softmax_bwd",
                     "b2n_norm_bwd_workspace_bytes", "b2n_strerror", "b2n_abi_version"):
        assert required in names


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(str(b200norm.LIB_PATH))
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, missing


def test_abi_version_and_strerror():
    lib = b200norm.load_library()
    assert lib.b2n_abi_version() == b200norm.ABI_VERSION
    assert lib.b2n_strerror(0) == b"ok"
    for code in range(-7, 0):
        assert lib.b2n_strerror(code) not in (b"ok", b"unknown status")
    assert lib.b2n_strerror(-99) == b"unknown status"


def test_argument_validation_needs_no_device():
    lib = b200norm.load_library()
    # negative sizes and bad enums are rejected before any CUDA call
    assert lib.b2n_layer_norm_fwd(None, None, None, None, None, None, -1, 8, 1e-5, 0, 0, None) == b200norm.ERR_BAD_ARG
    assert lib.b2n_layer_norm_fwd(None, None, None, None, None, None, 4, 8, 1e-5, 9, 0, None) == b200norm.ERR_BAD_ARG
    assert lib.b2n_softmax_fwd(None, None, 4, 8, 1, 0, 0, 0, None) == b200norm.ERR_BAD_ARG  # null pointers
    # empty problems are a successful no-op
    assert lib.b2n_layer_norm_fwd(None, None, None, None, None, None, 0, 8, 1e-5, 0, 0, None) == b200norm.OK
    assert lib.b2n_softmax_fwd(None, None, 0, 8, 1, 0, 0, 0, None) == b200norm.OK
    assert lib.b2n_nll_loss_fwd(None, None, None, None, None, None, None, 0, 4, 8, 5, -100, 0, 0, None) == b200norm.ERR_BAD_ARG


def test_path_forcing_round_trips():
    lib = b200norm.load_library()
    prev = lib.b2n_set_path(b200norm.PATH_RING)
    assert lib.b2n_set_path(prev) == b200norm.PATH_RING
    assert lib.b2n_set_path(77) == prev  # out-of-range values are ignored
    assert lib.b2n_set_path(prev) == prev


def test_aten_registration_is_built():
    assert b200norm.ATEN_LIB_PATH.exists()


def test_product_does_not_import_the_oracle():
    # the oracle is test infrastructure; nothing under the package or csrc may reference it
    pkg = ROOT / "torch-xpu-ops_b200"
    offenders = []
    for path in list(pkg.rglob("*.py")) + list(pkg.rglob("*.cu")) + list(pkg.rglob("*.cuh")) + list(pkg.rglob("*.cpp")) + list(pkg.rglob("*.h")):
        if "build" in path.parts:
            continue
        text = path.read_text()
        if re.search(r"^\s*(from|import)\s+oracle\b", text, flags=re.M) or "oracle/" in text:
            offenders.append(str(path))
    assert not offenders, offenders


def test_tuning_and_path_setters_validate_their_arguments():
    # host-side state only: no CUDA call is made
    lib = b200norm.load_library()
    for knob in (b200norm.TUNE_ROWS_PER_GROUP, b200norm.TUNE_STAGES, b200norm.TUNE_STORE_LAG,
                 b200norm.TUNE_CLUSTER_SIZE, b200norm.TUNE_SM_MARGIN):
        assert lib.b2n_set_tuning(knob, 2) == 0
        assert lib.b2n_set_tuning(knob, 0) == 0
        assert lib.b2n_set_tuning(knob, -1) == b200norm.ERR_BAD_ARG
    assert lib.b2n_set_tuning(99, 1) == b200norm.ERR_BAD_ARG
    prev = lib.b2n_set_path(b200norm.PATH_GENERIC)
    assert lib.b2n_set_path(1234) == b200norm.PATH_GENERIC   # an unknown family is ignored: the setting stays
    assert lib.b2n_set_path(prev) == b200norm.PATH_GENERIC


def test_entry_points_reject_bad_arguments_before_touching_the_device():
    lib = b200norm.load_library()
    bad = b200norm.ERR_BAD_ARG
    assert lib.b2n_layer_norm_fwd(None, None, None, None, None, None, -1, 8, 1e-5, 0, 0, None) == bad
    assert lib.b2n_layer_norm_fwd(None, None, None, None, None, None, 4, 8, 1e-5, 17, 0, None) == bad
    assert lib.b2n_layer_norm_fwd(None, None, None, None, None, None, 0, 8, 1e-5, 0, 0, None) == 0  # empty batch
    assert lib.b2n_softmax_fwd(None, None, 2, 4, 1, 0, 0, 3, None) == bad          # mode beyond safe softmax
    assert lib.b2n_softmax_fwd(None, None, 2, 4, 1, 0, 0, 0, None) == bad          # null pointers
    assert lib.b2n_masked_softmax_fwd(None, None, None, 2, 4, 0, 1, 0, None) == bad  # row_div < 1
    assert lib.b2n_cross_entropy_bwd(None, None, None, None, None, None, 3, 5, 7, -100, 0, 0, None) == bad  # reduction
    assert lib.b2n_cross_entropy_bwd(None, None, None, None, None, None, 0, 5, 1, -100, 0, 0, None) == 0


def test_spatial_softmax_tile_plans_keep_their_invariants():
    # The geometry of the tensor-map TMA tile kernels, computed on the host: a box row that is not a whole number
    # of 128-byte lines would put a bulk-tensor copy on a misaligned shared-memory address, and a team of threads
    # that is not whole warps would leave a named barrier short of arrivals -- neither may ever be planned.
    lib = b200norm.load_library()
    out = (ctypes.c_int * 8)()
    header, consumers, reg_rows = 1024 + 512 * 16, 512, 32
    seen_fit = seen_reg = seen_multibox = seen_nofit = 0
    for esize in (2, 4):
        cpt = 2 if esize == 2 else 1
        for backward in (0, 1):
            for n in (2, 3, 19, 31, 32, 33, 64, 100, 150, 255, 256, 257, 300, 700, 1000, 4096, 33000, 65536):
                for inner in (8, 64, 72, 136, 200, 512, 1000, 4096, 262144):
                    for outer in (1, 3, 16, 4096):
                        if (inner * esize) % 16:
                            continue
                        for smem in (232448, 101376):
                            rc = lib.b2n_softmax_tile_plan(outer, n, inner, esize, backward, 148, smem, out)
                            assert rc == 0
                            fits, w, nx, nb, stages, segs, reg, smem_used = list(out)
                            if not fits:
                                seen_nofit += 1
                                continue
                            seen_fit += 1
                            seen_reg += reg
                            seen_multibox += nx > 1
                            assert (w * esize) % 128 == 0 and 0 < w <= 256 and nx >= 1
                            assert nb == -(-n // -(-n // 256)) and nb <= 256   # boxes of equal height
                            groups = w * nx // cpt
                            assert groups % 32 == 0 and groups * segs <= consumers and segs >= 1
                            assert segs == 1 or groups // 32 <= 15          # named barriers 1..15
                            assert 2 <= stages <= 4 and header < smem_used <= smem
                            npad = -(-n // nb) * nb
                            assert smem_used == header + stages * npad * w * nx * esize * (2 if backward else 1)
                            if reg:
                                assert not backward and -(-n // segs) <= reg_rows
    assert seen_fit > 200 and seen_reg > 50 and seen_multibox > 20 and seen_nofit > 50
    assert lib.b2n_softmax_tile_plan(1, 4, 64, 3, 0, 148, 232448, out) != 0        # element size
    assert lib.b2n_softmax_tile_plan(1, 4, 64, 2, 0, 148, 232448, None) != 0       # no result array
