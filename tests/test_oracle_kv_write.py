"""CPU checks of the oracle's KV-write restatement (unpinned: the reference
kernel is CUDA-only): both pairings agree with a float64 complex rotation to
bf16 accuracy, untouched channels and skipped rows stay as they were."""
import numpy as np

import locks_oracle as orc


def _case(rot, seed=0):
    rng = np.random.default_rng(seed)
    n_tok, n_kv, d, page, NB, P = 4, 2, 128, 16, 5, 64
    key = orc.bf16_round(rng.standard_normal((n_tok, n_kv, d)).astype(np.float32))
    val = orc.bf16_round(rng.standard_normal((n_tok, n_kv, d)).astype(np.float32))
    ang = rng.uniform(0, 6.28, (P, rot // 2))
    cs = orc.bf16_round(np.concatenate([np.cos(ang), np.sin(ang)], 1).astype(np.float32))
    slots = np.array([17, -1, 3 * page + 15, 0], dtype=np.int64)
    pos = np.array([5, 6, 63, 0], dtype=np.int64)
    kc = np.full((NB, page, n_kv, d), 7.0, np.float32)
    vc = np.full((NB, page, n_kv, d), 7.0, np.float32)
    return key, val, kc, vc, slots, pos, cs, page


def test_rotation_matches_float64_both_pairings():
    for rot in (64, 128):
        for neox in (True, False):
            key, val, kc, vc, slots, pos, cs, page = _case(rot)
            orc.rope_and_cache(key, val, kc, vc, slots, pos, cs, rot, neox, page)
            half = rot // 2
            for r, s in enumerate(slots):
                if s < 0:
                    continue
                got = kc[s // page, s % page]
                c = cs[pos[r], :half].astype(np.float64)
                sn = cs[pos[r], half:rot].astype(np.float64)
                x = key[r].astype(np.float64)
                if neox:
                    e, o = x[:, :half], x[:, half:rot]
                    want = np.concatenate([e * c - o * sn, o * c + e * sn], 1)
                else:
                    want = np.empty_like(x[:, :rot])
                    want[:, 0::2] = x[:, 0:rot:2] * c - x[:, 1:rot:2] * sn
                    want[:, 1::2] = x[:, 1:rot:2] * c + x[:, 0:rot:2] * sn
                assert np.allclose(got[:, :rot], want, atol=0.02, rtol=0.01)
                assert np.array_equal(got[:, rot:], key[r][:, rot:])
                assert np.array_equal(vc[s // page, s % page], val[r])
                assert np.array_equal(got, orc.bf16_round(got))


def test_skipped_rows_and_other_slots_untouched():
    key, val, kc, vc, slots, pos, cs, page = _case(64, seed=3)
    orc.rope_and_cache(key, val, kc, vc, slots, pos, cs, 64, True, page)
    written = {(int(s) // page, int(s) % page) for s in slots if s >= 0}
    for b in range(kc.shape[0]):
        for t in range(page):
            if (b, t) not in written:
                assert (kc[b, t] == 7.0).all() and (vc[b, t] == 7.0).all()
    assert len(written) == 3
