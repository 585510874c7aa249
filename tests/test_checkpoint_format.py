"""Packed-checkpoint container (host side): a file written with the oracle's packing is read back by
`checkpoint.read_packed` with the layout documented in matmulfreellm_b200/checkpoint.py."""
import io
import json

import numpy as np
import pytest
import torch

from oracle import mmfree_oracle as O


def test_read_packed_parses_oracle_written_file(tmp_path):
    from matmulfreellm_b200 import checkpoint
    g = torch.Generator().manual_seed(0)
    w = torch.randn(200, 128, generator=g) * 0.02
    codes, mean = O.ternary_codes(w)
    packed = O.pack_ternary(codes)
    manifest = {"format": checkpoint.FORMAT_VERSION, "dtype": "float32", "bitlinear": {"lin": [200, 128]}, "tensors": {"emb": "float32"}}
    arrays = {
        "config.json": np.frombuffer(json.dumps({"hidden_size": 128}).encode(), dtype=np.uint8),
        "manifest.json": np.frombuffer(json.dumps(manifest).encode(), dtype=np.uint8),
        "lin.packed": packed.reshape(-1).view(np.uint8),
        "lin.scale": np.array([mean], dtype=np.float32),
        "lin.norm": np.ones(128, dtype=np.float32),
        "emb": np.zeros((4, 128), dtype=np.float32),
    }
    path = tmp_path / "t.npz"
    buf = io.BytesIO()
    np.savez(buf, **arrays)
    path.write_bytes(buf.getvalue())
    cfg, man, z = checkpoint.read_packed(str(path))
    assert cfg == {"hidden_size": 128} and man["bitlinear"]["lin"] == [200, 128]
    # 2 bits per weight, rows padded to whole 128-row tiles
    assert z["lin.packed"].nbytes == 2 * 128 * 128 // 4
    assert np.array_equal(z["lin.packed"].view(np.uint32), packed.reshape(-1))
    # a file of another format version is refused
    manifest["format"] = 99
    arrays["manifest.json"] = np.frombuffer(json.dumps(manifest).encode(), dtype=np.uint8)
    buf = io.BytesIO()
    np.savez(buf, **arrays)
    path.write_bytes(buf.getvalue())
    with pytest.raises(ValueError):
        checkpoint.read_packed(str(path))
