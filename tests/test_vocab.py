"""Move vocabulary and the 1858 -> 1929 mirror mapping: oracle pinned to the reference's lists by
digest, library pinned to the oracle entry by entry (integer/byte exact)."""
import ctypes

import numpy as np

from oracle import vocab


def test_oracle_lists_match_reference_digests():
    assert len(vocab.policy_leela) == 1858 and len(vocab.policy_index) == 1929
    assert vocab.digest(vocab.policy_leela) == vocab.SHA256_POLICY_LEELA
    assert vocab.digest(vocab.policy_index) == vocab.SHA256_POLICY_INDEX
    assert vocab.policy_index[:1858] == vocab.policy_leela
    assert vocab.policy_index[vocab.PAD_ID] == "padding_token"          # model_bis.py:173
    assert vocab.policy_leela[1792] == "a7a8q" and len(vocab.policy_index[1858:1924]) == 66


def test_known_answer_of_compare_policy_selftest():
    # Leela/compare_policy.py:526-545: one-hot at Leela index 4 in a White row lands on "a1f1",
    # one-hot at index 5 in a Black row lands on "a8g8"
    pol = np.zeros((255, 1858))
    pol[0, 4] = 1
    pol[1, 5] = 1
    out = vocab.map_leela_to_rl(pol, first_is_white=True)
    assert out.shape == (255, 1929) and out.dtype == np.float32
    assert vocab.policy_index.index("a1f1") == 4 and vocab.policy_index.index("a8g8") == 1619
    assert out[0, 4] == 1 and out[1, 1619] == 1 and out.sum() == 2


def test_mapping_black_is_injective_with_66_black_promotions():
    m = vocab.mapping_black
    assert len(set(m.tolist())) == 1858 and m.max() <= 1923 and int((m >= 1858).sum()) == 66


def test_knight_promotion_token():
    assert vocab.legal_token("a7a8n") == "a7a8" and vocab.legal_token("a7a8q") == "a7a8q"   # model_bis.py:376-379


def test_library_vocabulary_equals_oracle(lib):
    buf = ctypes.create_string_buffer(16)
    got = []
    for i in range(1929):
        assert lib.crl_vocab_move(i, buf) == 0
        got.append(buf.value.decode())
    assert got == vocab.policy_index
    assert lib.crl_vocab_move(1929, buf) < 0 and lib.crl_vocab_move(-1, buf) < 0
    mirror = [lib.crl_vocab_mirror_index(i) for i in range(1858)]
    assert mirror == vocab.mapping_black.tolist()
