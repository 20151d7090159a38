"""``install()`` rebinds the reference's by-name imports (needs a checkout of the reference; skipped without one)."""

from __future__ import annotations

import os
import sys
import tempfile
from pathlib import Path

import pytest

# A checkout of the reference: MIE_REFERENCE_CHECKOUT, else a directory named "reference" beside this repository.
REFERENCE = Path(os.environ.get("MIE_REFERENCE_CHECKOUT", str(Path(__file__).resolve().parents[2] / "reference")))


@pytest.mark.skipif(not (REFERENCE / "engine" / "kv_cache").is_dir(), reason="no reference checkout on this host")
def test_install_rebinds_every_importing_module():
    link_dir = Path(tempfile.mkdtemp(prefix="minillm_ref_"))
    (link_dir / "minillm_l4").symlink_to(REFERENCE)
    sys.path.insert(0, str(link_dir))
    try:
        import minillm_l4  # noqa: F401
        import minillm_l4.engine.kv_cache.paged_attention  # noqa: F401
        import minillm_l4.engine.kv_cache.qwen3_paged  # noqa: F401

        from mini_inference_engine_b200 import install

        paged = sys.modules["minillm_l4.engine.kv_cache.paged_attention"]
        adapter = sys.modules["minillm_l4.engine.kv_cache.qwen3_paged"]
        package = sys.modules["minillm_l4.engine.kv_cache"]
        before = paged.triton_paged_decode_attention
        assert install.install(sys.modules["minillm_l4"]) > 20
        ours = "mini_inference_engine_b200.engine"
        assert paged.triton_paged_decode_attention.__module__.startswith(ours)
        assert paged.can_use_triton_paged_decode.__module__.startswith(ours)
        assert adapter.triton_write_decode_kv.__module__.startswith(ours)
        assert adapter.triton_write_packed_kv.__module__.startswith(ours)
        assert adapter.project_qkv.__module__.startswith(ours)
        assert adapter.validate_decode_metadata.__module__.startswith(ours)
        assert package.select_decode_split_count.__module__.startswith(ours)
        assert sys.modules["minillm_l4.engine.kernels"].sm89_fp8_linear.__module__.startswith(ours)
        install.uninstall()
        assert paged.triton_paged_decode_attention is before
    finally:
        sys.path.remove(str(link_dir))
