"""TEST INFRASTRUCTURE ONLY - not part of the product; imported by tests/ alone.

CPU restatement (numpy, exact uint32 arithmetic) of the device-side draws of myea_b200/csrc/masks.cu, which replace the
reference's host-side generators (Neural_Network__Dropout__Bernoulli__Loop.cpp:70-90,
Neural_Network__Dropout__Zoneout__Loop.cpp:57-100, Neural_Network__Forward_Pass__Loop.cpp:5016-5045: one std::mt19937
walk per mask).  The reference's streams cannot be reproduced by a parallel generator, so parity for this row is:
 * the generator itself against the published known-answer vectors of Philox4x32-10 (Salmon et al., SC'11; the vectors
   ship with the authors' Random123 distribution) - pinned in tests/test_masks_cpu.py;
 * the device arrays against this restatement, bit for bit;
 * the arrays' statistics against the probabilities the reference passes to its generators.
"""
import numpy as np

M0, M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
W0, W1 = 0x9E3779B9, 0xBB67AE85
MASK = np.uint64(0xFFFFFFFF)

KIND_BERNOULLI, KIND_ZONEOUT_STATE, KIND_ZONEOUT_OUTPUT, KIND_SHAKEDROP, KIND_SHAKEDROP_ALPHA, KIND_SHAKEDROP_BETA = range(6)


def philox4x32_10(counter, key):
    """counter: [..., 4] uint32, key: (k0, k1) -> [..., 4] uint32"""
    c = [np.asarray(counter[..., i], np.uint64) for i in range(4)]
    k0, k1 = int(key[0]) & 0xFFFFFFFF, int(key[1]) & 0xFFFFFFFF
    for _ in range(10):
        p0, p1 = M0 * c[0], M1 * c[2]
        hi0, lo0, hi1, lo1 = p0 >> np.uint64(32), p0 & MASK, p1 >> np.uint64(32), p1 & MASK
        c = [hi1 ^ c[1] ^ np.uint64(k0), lo1, hi0 ^ c[3] ^ np.uint64(k1), lo0]
        k0, k1 = (k0 + W0) & 0xFFFFFFFF, (k1 + W1) & 0xFFFFFFFF
    return np.stack([x.astype(np.uint32) for x in c], axis=-1)


def uniform(seed, step, layer, kind, n):
    """the first n draws of stream (layer, kind) at (seed, step): float32 in [0, 1)"""
    blocks = (n + 3) // 4
    ctr = np.zeros((blocks, 4), np.uint32)
    ctr[:, 0] = np.arange(blocks, dtype=np.uint64).astype(np.uint32)
    ctr[:, 1] = np.uint32(step & 0xFFFFFFFF)
    ctr[:, 2] = np.uint32((step >> 32) & 0xFFFFFFFF)
    ctr[:, 3] = np.uint32(8 * layer + kind)
    words = philox4x32_10(ctr, (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)).reshape(-1)[:n]
    return (words >> np.uint32(8)).astype(np.float32) * np.float32(1.0 / 16777216.0)


def bernoulli_mask(seed, step, layer, n, retention):
    return (uniform(seed, step, layer, KIND_BERNOULLI, n) < np.float32(retention)).astype(np.uint8)


def zoneout_masks(seed, step, layer, n, p_state, p_output):
    """[T][dirs*cells] numbering; 1 = compute, 0 = keep the previous value"""
    return ((uniform(seed, step, layer, KIND_ZONEOUT_STATE, n) >= np.float32(p_state)).astype(np.uint8),
            (uniform(seed, step, layer, KIND_ZONEOUT_OUTPUT, n) >= np.float32(p_output)).astype(np.uint8))


def shakedrop(seed, step, layer, batch, width, p):
    mask = (uniform(seed, step, layer, KIND_SHAKEDROP, batch) < np.float32(p)).astype(np.uint8)
    u = uniform(seed, step, layer, KIND_SHAKEDROP_ALPHA, batch * width)
    alpha = (np.float32(2.0) * u + np.float32(-1.0)).astype(np.float32).reshape(batch, width)   # 2u is exact: one rounding, as the device fma
    beta = uniform(seed, step, layer, KIND_SHAKEDROP_BETA, batch * width).reshape(batch, width)
    return mask, alpha, beta
