"""The C-ABI library: every symbol the header declares is exported, and the host-side
argument checks answer without a GPU (no compute call is made here)."""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest

from fusedindextopk_b200 import _lib
from fusedindextopk_b200.build import build

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "itk_b200.h"


@pytest.fixture(scope="module")
def library():
    build()
    return _lib.load_library()


def declared_functions() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(itk_[a-z0-9_]+)\s*\(", text)))


def test_header_and_loader_agree(library):
    names = declared_functions()
    assert names, "no declarations found in the header"
    assert set(names) == set(_lib.EXPORTED_SYMBOLS)
    for name in names:
        assert getattr(library, name) is not None


def test_version_and_constants(library):
    assert "sm_100a" in _lib.version()
    header = HEADER.read_text()
    for macro, value in (("ITK_TOP_K", _lib.TOP_K), ("ITK_BLOCK_Q", _lib.BLOCK_Q),
                         ("ITK_REPAIR_CHUNK", _lib.REPAIR_CHUNK), ("ITK_SPILL_U64_PER_ROW", _lib.SPILL_U64_PER_ROW),
                         ("ITK_MAX_KEYS", _lib.MAX_KEYS), ("ITK_MAX_PAIR_SOURCES", _lib.MAX_PAIR_SOURCES),
                         ("ITK_MAX_CTAS", _lib.MAX_CTAS)):
        assert re.search(rf"#define {macro} {value}\b", header), macro


def test_workspace_sizes_need_no_gpu(library):
    sizes = _lib.workspace_sizes(4096, 16384, 1)
    # one spill region per CTA and unit row: capped at 4 x ITK_MAX_CTAS regions, never more than the units need
    assert sizes.spill_bytes == 4 * _lib.MAX_CTAS * _lib.SPILL_U64_PER_ROW * 8
    assert _lib.workspace_sizes(10, 16384, 1).spill_bytes == 12 * _lib.SPILL_U64_PER_ROW * 8
    assert _lib.workspace_sizes(10, 16384, 4).spill_bytes == 48 * _lib.SPILL_U64_PER_ROW * 8
    assert sizes.repair_pairs_bytes == 4096 * 16384 * 8
    assert sizes.pairs_bytes == 4096 * 2048 * 8
    assert sizes.repair_chunks == 1
    assert _lib.workspace_sizes(64, 163840, 1).repair_chunks == 10
    with pytest.raises(_lib.ItkError, match="shards"):
        _lib.workspace_sizes(8, 8192, 99)


def test_argument_errors_are_reported_before_any_launch(library):
    args = _lib.FusedArgs()
    status = library.itk_fused_topk(ctypes.byref(args), None)
    assert status == -1
    assert b"must not be null" in library.itk_last_error()
    assert library.itk_gather_sampled_kv(None, None, None, None, None, 8, 4, None) == -1
    assert library.itk_update_chunk_ranges(None, None, None, None, 4, 8192, None) == -1
    assert library.itk_merge_candidate_lists(None, None, 2, None, None, None, 4, None) == -1
    # the entry points of the repair stage
    assert library.itk_compact_flagged_rows(None, None, None, None, None, 8, 32, None, None, None, None, None, None) == -1
    assert b"must not be null" in library.itk_last_error()
    body = ctypes.c_void_p()
    assert library.itk_flagged_scope_begin(None, 8, None, ctypes.byref(body)) == -1
    assert library.itk_flagged_scope_end(None, None) == 0      # nothing was opened: nothing to close
    assert library.itk_repair_merge_chunk(None, None, None, None, None, 0, 16384, None, None, 8, 1, 1,
                                          None, None, None, None, None) == -1
    assert library.itk_merge_shard_lists(None, None, 17, None, None, None, 4, None, None, None, None, 0, 0,
                                         0, 1, 0, None, None, None) == -1


def test_fused_args_layout_matches_header():
    """Field order of the ctypes mirror follows the struct in the header."""

    text = HEADER.read_text()
    body = text[text.index("typedef struct itk_fused_args {"):text.index("} itk_fused_args;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = re.findall(r"\b([a-z_0-9]+);", body)
    assert fields == [name for name, _ in _lib.FusedArgs._fields_]
