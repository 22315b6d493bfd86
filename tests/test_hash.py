"""OaFnHash against hashlib (SHAKE) and a host Keccak-f[1600]; the device kernels against the same oracles."""
import hashlib

import numpy as np
import pytest
import torch

from oa_b200.core.matrix import OaMatrix
from oa_b200.crypto import fn_hash as H


def _shake_by_permutation(msg: bytes, out_len: int, rate: int) -> bytes:
    """SHAKE built from the host permutation: checks keccak_f1600_host against hashlib."""
    st = bytearray(200)
    pos = 0
    for b in msg:
        st[pos] ^= b
        pos += 1
        if pos == rate:
            st = bytearray(H.keccak_f1600_host(np.frombuffer(bytes(st), "<u8").reshape(1, 25)).astype("<u8").tobytes())
            pos = 0
    st[pos] ^= 0x1F
    st[rate - 1] ^= 0x80
    out = b""
    while len(out) < out_len:
        st = bytearray(H.keccak_f1600_host(np.frombuffer(bytes(st), "<u8").reshape(1, 25)).astype("<u8").tobytes())
        out += bytes(st[:rate])
    return out[:out_len]


def test_host_permutation_reproduces_shake():
    for n, out_len in ((0, 32), (5, 16), (136, 32), (300, 200)):
        msg = bytes((i * 7 + 3) & 0xFF for i in range(n))
        assert _shake_by_permutation(msg, out_len, 136) == hashlib.shake_256(msg).digest(out_len)
        assert _shake_by_permutation(msg, out_len, 168) == hashlib.shake_128(msg).digest(out_len)


def _check(device):
    g = torch.Generator().manual_seed(0)
    for rows, msg_len, out_len in ((7, 33, 32), (300, 136, 32), (4, 400, 200), (5, 1, 5)):
        msg = torch.randint(0, 256, (rows, msg_len), generator=g, dtype=torch.uint8)
        for bits, fn, h in ((256, H.Shake256, hashlib.shake_256), (128, H.Shake128, hashlib.shake_128)):
            out = fn(OaMatrix(msg.to(device)), out_len).Tensor().cpu()
            assert out.shape == (rows, (out_len + 7) // 8 * 8)
            for i in (0, rows - 1):
                assert bytes(out[i, :out_len].tolist()) == h(bytes(msg[i].tolist())).digest(out_len), (bits, rows, msg_len)
            assert out[:, out_len:].sum() == 0
    st = torch.randint(0, 256, (65, 200), generator=g, dtype=torch.uint8)
    got = H.KeccakF1600(OaMatrix(st.to(device))).Tensor().cpu()
    want = H.keccak_f1600_host(np.frombuffer(st.numpy().tobytes(), "<u8").reshape(-1, 25)).astype("<u8").tobytes()
    assert got.numpy().tobytes() == want
    leaves = torch.randint(0, 256, (64, 32), generator=g, dtype=torch.uint8)
    root = H.MerkleRoot(OaMatrix(leaves.to(device))).Tensor().cpu()
    assert root.shape == (1, 32) and bytes(root[0].tolist()) == H.OaMerkleRoot([bytes(r.tolist()) for r in leaves])
    one = H.MerkleRoot(OaMatrix(leaves[:1].to(device))).Tensor().cpu()
    assert torch.equal(one, leaves[:1])
    with pytest.raises(ValueError):
        H.MerkleRoot(OaMatrix(leaves[:3].to(device)))


def test_fn_hash_cpu():
    _check("cpu")
    assert H.OaMerkleRoot([]) == bytes(32)
    a, b, c = (bytes([i]) * 32 for i in (1, 2, 3))
    assert H.OaMerkleRoot([a, b, c]) == H.OaHashCombine(H.OaHashCombine(a, b), H.OaHashCombine(c, c))


@pytest.mark.gpu
def test_fn_hash_kernels():
    from oa_b200.ops import kernels as K
    _check("cuda")
    K.check_status()
