"""Paged radix tree against a naive model: random sequences of add / extend / fork / rollback /
remove / match are replayed on the native tree and on a dict of plain token lists, and every
observable (tokens, lengths, membership, longest-prefix matches, free capacity at quiescence) must
agree.  Interface parity: ``cpp/serve/radix_tree.h`` of the reference (add / extend / fork / rollback /
remove / match / free capacity)."""
import random

import pytest

from mlc_llm_b200._core import PagedRadixTree


class NaiveTree:
    """Sequences as plain lists; a prefix match is a linear scan."""

    def __init__(self):
        self.seqs = {}

    def match(self, tokens):
        best, ids = 0, []
        for sid, seq in self.seqs.items():
            n = 0
            while n < len(seq) and n < len(tokens) and seq[n] == tokens[n]:
                n += 1
            if n > best:
                best, ids = n, [sid]
            elif n == best and n > 0:
                ids.append(sid)
        return best, set(ids)


def _lcp_alphabet(rng):
    # a two-letter alphabet makes shared prefixes (and therefore node splits) the common case
    return rng.choice([(1, 2), (1, 2, 3), tuple(range(1, 40))])


def _check_all(tree, model):
    for sid, seq in model.seqs.items():
        assert tree.has(sid)
        assert tree.get_length(sid) == len(seq)
        assert list(tree.get(sid)) == seq


@pytest.mark.parametrize("seed", range(12))
def test_random_operations_agree_with_the_naive_model(seed):
    rng = random.Random(seed)
    alphabet = _lcp_alphabet(rng)
    tree, model = PagedRadixTree(), NaiveTree()
    capacity = tree.free_capacity()
    next_id = 0
    for step in range(400):
        live = list(model.seqs)
        op = rng.choice(["add", "extend", "extend", "fork", "rollback", "remove", "match", "match"])
        if op == "add" or not live:
            tree.add(next_id)
            model.seqs[next_id] = []
            next_id += 1
        elif op == "extend":
            sid = rng.choice(live)
            # lengths straddle the tree's internal block size now and then
            n = rng.choice([1, 2, 5, 17, 64, 65, 130])
            toks = [rng.choice(alphabet) for _ in range(n)]
            tree.extend(sid, toks)
            model.seqs[sid] += toks
        elif op == "fork":
            parent = rng.choice(live)
            at = rng.randint(0, len(model.seqs[parent]))
            tree.fork(next_id, parent, at)
            model.seqs[next_id] = list(model.seqs[parent][:at])
            next_id += 1
        elif op == "rollback":
            sid = rng.choice(live)
            if model.seqs[sid]:
                n = rng.randint(1, len(model.seqs[sid]))
                tree.rollback(sid, n)
                del model.seqs[sid][-n:]
        elif op == "remove":
            sid = rng.choice(live)
            tree.remove(sid)
            del model.seqs[sid]
            assert not tree.has(sid)
        else:
            base = list(model.seqs[rng.choice(live)]) if rng.random() < 0.8 else []
            cut = rng.randint(0, len(base))
            query = base[:cut] + [rng.choice(alphabet) for _ in range(rng.randint(0, 6))]
            got_len, got_ids = tree.match(query)
            want_len, want_ids = model.match(query)
            assert got_len == want_len, (step, query)
            assert set(got_ids) == want_ids, (step, query)
        if step % 25 == 0:
            _check_all(tree, model)
    _check_all(tree, model)
    for sid in list(model.seqs):
        tree.remove(sid)
    assert tree.free_capacity() == capacity   # every block went back to the pool


def test_shared_prefixes_are_stored_once():
    tree = PagedRadixTree()
    tree.add(0)
    tree.extend(0, [7] * 300)
    used_one = tree.free_capacity()
    for sid in range(1, 9):
        tree.fork(sid, 0, 300)
    assert tree.free_capacity() == used_one           # forks at the tip cost nothing
    tree.extend(3, [8] * 10)
    assert tree.free_capacity() < used_one            # a divergent tail does
    assert list(tree.get(3)) == [7] * 300 + [8] * 10
    assert list(tree.get(4)) == [7] * 300


def test_fork_in_the_middle_then_diverge():
    tree = PagedRadixTree()
    tree.add(0)
    tree.extend(0, [0, 1, 2, 3])
    tree.fork(1, 0, 3)
    tree.extend(1, [4])
    assert list(tree.get(0)) == [0, 1, 2, 3] and list(tree.get(1)) == [0, 1, 2, 4]
    n, ids = tree.match([0, 1, 2, 4, 9])
    assert n == 4 and set(ids) == {1}
    n, ids = tree.match([0, 1, 2])
    assert n == 3 and set(ids) == {0, 1}
    tree.rollback(1, 2)
    assert list(tree.get(1)) == [0, 1] and list(tree.get(0)) == [0, 1, 2, 3]


def test_capacity_is_bounded_and_reported():
    tree = PagedRadixTree(4)
    start = tree.free_capacity()
    tree.add(0)
    tree.extend(0, [1] * (start // 2))
    assert 0 < tree.free_capacity() < start
    tree.remove(0)
    assert tree.free_capacity() == start
