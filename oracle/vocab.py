"""Move vocabularies of the reference, restated as a generator (TEST INFRASTRUCTURE: only tests,
the smoke check and the bench's CPU baseline may import this package).

The reference stores two literal lists (utils/vocab.py:9-227 `policy_index`, 229-438 `policy_leela`;
identical copies in Leela/vocab.py, Leela/gen_TC.py:321-530, Leela/compare_policy.py:2-432):

* `policy_leela` (1858 entries): for every from-square in a1,b1,...,h1,a2,...,h8 order, every
  to-square in the same order that a queen or a knight could reach; then the 66 white promotions
  (from rank 7, file a..h; capture-left, push, capture-right; pieces q, r, b - a knight promotion is
  the plain 4-character move).
* `policy_index` (1929 entries): `policy_leela`, then the 66 black promotions (rank 2 -> 1) in the
  same order, then 5 special tokens; id 1928 is the padding token (model_bis.py:173,194).

The sha256 digests below pin this restatement to the reference's lists (joined with newlines).
"""
import hashlib

import numpy as np

FILES = "abcdefgh"
SPECIAL_TOKENS = ["<thinking>", "</thinking>", "end_variation", "end", "padding_token"]
SHA256_POLICY_LEELA = "4a901f49851725496e39e34648dd58f240950fa6b72a0bbf6b2816b9af767cc7"
SHA256_POLICY_INDEX = "4f88911e08f3d3959eb86e060b6f51af4eb3a17fbdd1dd63acfdf2223d36148c"
PAD_ID = 1928


def _sq_name(sq):
    return FILES[sq % 8] + str(sq // 8 + 1)


def _reachable(frm, to):
    if frm == to:
        return False
    df, dr = abs(frm % 8 - to % 8), abs(frm // 8 - to // 8)
    return df == 0 or dr == 0 or df == dr or (df, dr) in ((1, 2), (2, 1))


def _promotions(from_rank, to_rank):
    out = []
    for f in range(8):
        for tf in (f - 1, f, f + 1):
            if 0 <= tf < 8:
                for piece in "qrb":
                    out.append(f"{FILES[f]}{from_rank}{FILES[tf]}{to_rank}{piece}")
    return out


def build_policy_leela():
    moves = [_sq_name(a) + _sq_name(b) for a in range(64) for b in range(64) if _reachable(a, b)]
    return moves + _promotions(7, 8)


def build_policy_index():
    return build_policy_leela() + _promotions(2, 1) + list(SPECIAL_TOKENS)


policy_leela = build_policy_leela()
policy_index = build_policy_index()


def digest(moves):
    return hashlib.sha256("\n".join(moves).encode()).hexdigest()


def mirror_uci(uci):
    """Flip ranks 1<->8 of a 4- or 5-character UCI move (Leela/compare_policy.py:437-463)."""
    tail = uci[4:] if len(uci) == 5 else ""
    return f"{uci[0]}{9 - int(uci[1])}{uci[2]}{9 - int(uci[3])}{tail}"


def build_mapping_black():
    """Leela index -> index in `policy_index` of the rank-mirrored move (compare_policy.py:465-483)."""
    lookup = {m: i for i, m in enumerate(policy_index)}
    return np.array([lookup[mirror_uci(m)] for m in policy_leela], dtype=np.int32)


mapping_black = build_mapping_black()


def map_leela_to_rl(policies, first_is_white=True):
    """[B,1858] -> zero-filled [B,1929] f32; rows alternate White (identity) / Black (mirror scatter)
    starting with White when `first_is_white` (compare_policy.py:493-523)."""
    policies = np.asarray(policies)
    if policies.shape[1] != len(policy_leela):
        raise ValueError("expected 1858 columns")
    res = np.zeros((policies.shape[0], len(policy_index)), dtype=np.float32)
    rows = np.arange(policies.shape[0])
    white = rows[(rows % 2 == 0) == bool(first_is_white)]
    black = rows[(rows % 2 == 0) != bool(first_is_white)]
    res[np.ix_(white, np.arange(len(policy_leela)))] = policies[white]
    res[np.ix_(black, mapping_black)] = policies[black]
    return res


def move_squares(uci):
    """(from, to, promo) with a1 = 0, b1 = 1, ..., h8 = 63; promo in {0: none, 1: q, 2: r, 3: b}."""
    frm = FILES.index(uci[0]) + 8 * (int(uci[1]) - 1)
    to = FILES.index(uci[2]) + 8 * (int(uci[3]) - 1)
    promo = 0 if len(uci) == 4 else " qrb".index(uci[4])
    return frm, to, promo


def legal_token(uci):
    """Vocabulary string of a legal move: knight promotions drop the 'n' (model_bis.py:376-379)."""
    return uci[:-1] if uci.endswith("n") else uci


def choose_moves(rows, is_prob, temperature, uniforms=None):
    """Test oracle for the on-device move choice (model_bis.py:385-394: temperature 0 -> arg-max, else a draw from
    softmax(logits / T); the draw is made reproducible by taking the caller's uniform number through the
    inverse CDF). rows: [B, V] logits, or probabilities with is_prob. Returns (index [B], margin [B]) where
    margin is the relative distance of u * total from the nearest CDF step (a caller comparing against
    another implementation may accept a neighbouring index when the margin is within rounding)."""
    import numpy as np
    rows = np.asarray(rows, dtype=np.float32)
    B = rows.shape[0]
    best = rows.argmax(axis=1)
    if uniforms is None or temperature == 0:
        return best.astype(np.int32), np.ones(B)
    inv_t = np.float32(1.0 / temperature)
    top = rows.max(axis=1, keepdims=True)
    if is_prob:
        w = np.where(rows > 0, np.power(np.maximum(rows, 0) / top, inv_t, dtype=np.float32), np.float32(0))
    else:
        w = np.exp((rows - top) * inv_t, dtype=np.float32)
    cdf = np.cumsum(w.astype(np.float64), axis=1)
    thr = np.asarray(uniforms, dtype=np.float32).astype(np.float64) * cdf[:, -1]
    idx = (cdf > thr[:, None]).argmax(axis=1)
    none = ~(cdf > thr[:, None]).any(axis=1)
    idx[none] = best[none]
    margin = np.abs(cdf - thr[:, None]).min(axis=1) / cdf[:, -1]
    return idx.astype(np.int32), margin
