"""ML-DSA-65 (FIPS 204): sizes, number-theoretic transform, round trip, rejection of altered inputs, and interoperability
with the OpenSSL implementation when the `cryptography` package offers it (used as an oracle only).
Reference surface: Source/Public/Oa/Crypto/Sign.h; its tests are Test/Crypto/TestSign.cpp."""
import pytest
import torch

from oa_b200.crypto import sign as S


def test_sizes_and_constants():
    assert (S.OA_SIGN_PUBKEY_SIZE, S.OA_SIGN_SECRET_SIZE, S.OA_SIGN_SIG_SIZE) == (1952, 4032, 3309)
    assert S._ZETAS[1] == pow(1753, 128, S.Q) and (S._INV256 * 256) % S.Q == 1 and pow(1753, 512, S.Q) == 1 and pow(1753, 256, S.Q) == S.Q - 1


def test_ntt_is_the_negacyclic_convolution():
    torch.manual_seed(0)
    a, b = torch.randint(0, S.Q, (4, 3, 256)), torch.randint(0, S.Q, (4, 3, 256))
    assert torch.equal(S.NttInverse(S.Ntt(a)), a)                                      # batched, any leading shape
    x, y = a[0, 0], b[0, 0]
    want = [0] * 256
    xs, ys = x.tolist(), y.tolist()
    for i in range(256):
        for j in range(256):
            k = i + j
            if k < 256:
                want[k] = (want[k] + xs[i] * ys[j]) % S.Q
            else:
                want[k - 256] = (want[k - 256] - xs[i] * ys[j]) % S.Q
    assert S.NttInverse(S._mul(S.Ntt(x), S.Ntt(y))).tolist() == want


def test_packing_and_hints_round_trip():
    torch.manual_seed(1)
    w = torch.randint(-S.ETA, S.ETA + 1, (256,))
    assert torch.equal(S._bit_unpack(S._bit_pack(w, S.ETA, S.ETA), S.ETA, S.ETA), w) and len(S._bit_pack(w, S.ETA, S.ETA)) == 128
    z = torch.randint(-(S.GAMMA1 - 1), S.GAMMA1 + 1, (256,))
    assert torch.equal(S._bit_unpack(S._bit_pack(z, S.GAMMA1 - 1, S.GAMMA1), S.GAMMA1 - 1, S.GAMMA1), z)
    h = torch.zeros(S.K_ROWS, 256, dtype=torch.int64)
    h[0, [3, 77]] = 1
    h[4, 255] = 1
    assert torch.equal(S._hint_unpack(S._hint_pack(h)), h)
    bad = bytearray(S._hint_pack(h))
    bad[0], bad[1] = bad[1], bad[0]                                                    # indices no longer increasing
    assert S._hint_unpack(bytes(bad)) is None
    r = torch.randint(0, S.Q, (1000,))
    r1, r0 = S._decompose(r)
    assert torch.equal((r1 * 2 * S.GAMMA2 + r0) % S.Q, r) and int(r0.abs().max()) <= S.GAMMA2 and int(r1.max()) <= 15
    t1, t0 = S._power2round(r)
    assert torch.equal((t1 << S.D) + t0, r) and int(t0.abs().max()) <= 1 << (S.D - 1)
    c = S._sample_in_ball(bytes(range(48)))
    assert int(c.abs().sum()) == S.TAU and set(c.tolist()) <= {-1, 0, 1}


def test_sign_verify_round_trip_and_rejections():
    kp = S.OaGenerateKeypair(bytes(range(32)))
    again = S.OaGenerateKeypair(bytes(range(32)))
    assert kp.Public == again.Public and kp.Secret.Bytes == again.Secret.Bytes and not kp.Public.IsZero()
    assert len(kp.Public.Bytes) == 1952 and len(kp.Secret.Bytes) == 4032 and len(kp.Public.ToShortHex()) == 32
    msg = b"the quick brown fox"
    det = S.OaSign(kp.Secret, msg, deterministic=True)
    assert det == S.OaSign(kp.Secret, msg, deterministic=True) and len(det.Bytes) == 3309
    hedged = S.OaSign(kp.Secret, msg)
    assert hedged != det and S.OaVerify(kp.Public, msg, hedged) and S.OaVerify(kp.Public, msg, det)
    assert not S.OaVerify(kp.Public, msg + b"!", det)
    assert not S.OaVerify(kp.Public, msg, det, ctx=b"other context")
    with_ctx = S.OaSign(kp.Secret, msg, ctx=b"oa", deterministic=True)
    assert S.OaVerify(kp.Public, msg, with_ctx, ctx=b"oa") and not S.OaVerify(kp.Public, msg, with_ctx)
    flipped = bytearray(det.Bytes)
    flipped[100] ^= 1
    assert not S.OaVerify(kp.Public, msg, S.OaSignature(bytes(flipped)))
    assert not S.OaVerify(S.OaGenerateKeypair(bytes(32)).Public, msg, det)
    assert not S.OaVerify(kp.Public, msg, S.OaSignature(det.Bytes[:-1]))
    kp.Secret.SecureZero()
    assert kp.Secret.IsZero()
    with pytest.raises(ValueError):
        S.OaSign(kp.Secret, msg)
    with pytest.raises(ValueError):
        S.OaGenerateKeypair(b"short")


def test_interoperates_with_openssl():
    mldsa = pytest.importorskip("cryptography.hazmat.primitives.asymmetric.mldsa")
    seed = bytes(range(100, 132))
    try:
        ref = mldsa.MLDSA65PrivateKey.from_seed_bytes(seed)
    except Exception as e:                    # a build of the package without ML-DSA in its OpenSSL
        pytest.skip(f"ML-DSA not available in this cryptography build: {e}")
    kp = S.OaGenerateKeypair(seed)
    assert ref.public_key().public_bytes_raw() == kp.Public.Bytes                      # same key from the same seed
    msg = b"interoperability"
    ref.public_key().verify(S.OaSign(kp.Secret, msg).Bytes, msg)                        # raises on a bad signature
    assert S.OaVerify(kp.Public, msg, S.OaSignature(ref.sign(msg)))
    ref.public_key().verify(S.OaSign(kp.Secret, msg, ctx=b"ctx").Bytes, msg, b"ctx")
    assert S.OaVerify(kp.Public, msg, S.OaSignature(ref.sign(msg, b"ctx")), ctx=b"ctx")
