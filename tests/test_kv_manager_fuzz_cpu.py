"""Paged KV manager against a shadow of the device memory: random adds, forks at arbitrary positions, chunked and
tree appends, tree commits, roll-backs, windows and removals. The shadow applies every plan the way the model side
does (page copies first, then the appended rows, token moves gathered before they are written); after every
forward each sequence must read back exactly its own history through its page table, and no page may leak."""
import numpy as np
import pytest

from mlc_llm_b200 import _core

PAGE = 16


class Shadow:
    def __init__(self, num_pages, max_seqs, seed):
        self.kv = _core.KVManager(num_pages, PAGE, max_seqs)
        self.num_pages = num_pages
        self.mem = np.full(num_pages * PAGE, -1, dtype=np.int64)
        self.want = {}            # sequence -> tags of its positions
        self.window = {}          # sequence -> (window, sink)
        self.rng = np.random.default_rng(seed)
        self.next_tag = 0
        self.next_id = 0

    def apply(self, plan):
        # the device copies all pairs of a plan in one launch: every source is read before any destination is
        # written here, and a destination that is also another pair's source is reported
        copies = np.asarray(plan["page_copies"]).reshape(-1, 2).tolist()
        assert not ({d for _, d in copies} & {s for s, _ in copies}), ("a pair writes what another reads", copies)
        assert len({d for _, d in copies}) == len(copies), ("two pairs write one page", copies)
        rows = [self.mem[src * PAGE:(src + 1) * PAGE].copy() for src, _ in copies]
        for (_, dst), row in zip(copies, rows):
            self.mem[dst * PAGE:(dst + 1) * PAGE] = row
        tags = np.arange(self.next_tag, self.next_tag + len(plan["slots"]))
        self.next_tag += len(tags)
        self.mem[np.asarray(plan["slots"], dtype=np.int64)] = tags
        return tags

    def check(self):
        held = set()
        for sid, want in self.want.items():
            pages = self.kv.sequence_pages(sid)
            assert self.kv.sequence_length(sid) == len(want)
            held.update(p for p in pages if p >= 0)
            win, sink = self.window.get(sid, (0, 0))
            first = 0 if win == 0 else max(0, len(want) - win + 1)
            for pos in list(range(min(sink, len(want)))) + list(range(first, len(want))):
                pg = pages[pos // PAGE]
                assert pg >= 0, (sid, pos, "a visible position lost its page")
                assert self.mem[pg * PAGE + pos % PAGE] == want[pos], (sid, pos)
        assert len(held) == self.num_pages - self.kv.num_available_pages(), "page accounting"

    # ------------------------------------------------------------------ operations
    def add(self):
        sid = self.next_id
        self.next_id += 1
        self.kv.add_sequence(sid)
        self.want[sid] = []
        if self.rng.random() < 0.3:
            win, sink = int(self.rng.integers(20, 60)), int(self.rng.integers(0, 6))
            self.kv.enable_sliding_window(sid, win, sink)
            self.window[sid] = (win, sink)

    def forward(self):
        ids = [s for s in self.want if self.rng.random() < 0.6]
        if not ids:
            return
        lens = [int(self.rng.integers(1, 40)) for _ in ids]
        try:
            plan = self.kv.begin_forward(ids, lens)
        except RuntimeError:
            return                      # out of pages: nothing may have changed
        tags = self.apply(plan)
        off = 0
        for sid, n in zip(ids, lens):
            self.want[sid].extend(tags[off:off + n].tolist())
            off += n
        self.check()

    def tree(self):
        ids = [s for s in self.want if self.window.get(s, (0, 0))[0] == 0]
        if not ids:
            return
        sid = ids[int(self.rng.integers(0, len(ids)))]
        n = int(self.rng.integers(2, 12))
        parents = [-1] + [int(self.rng.integers(-1, j)) for j in range(1, n)]
        try:
            plan = self.kv.begin_forward([sid], [n], parents)
        except RuntimeError:
            return
        tags = self.apply(plan).tolist()
        # accept a root-to-leaf path: increasing node indices
        path, node = [], int(self.rng.integers(0, n))
        while node >= 0:
            path.append(node)
            node = parents[node]
        accepted = sorted(path)[: int(self.rng.integers(0, len(path) + 1))]
        moves = np.asarray(self.kv.commit_tree_nodes(sid, n, accepted), dtype=np.int64).reshape(-1, 2)
        if len(moves):
            vals = self.mem[moves[:, 0]].copy()
            self.mem[moves[:, 1]] = vals
        self.want[sid].extend(tags[a] for a in accepted)
        plan = self.kv.begin_forward([sid], [1])        # delivers a copy the roll-back may have queued
        self.want[sid].append(int(self.apply(plan)[0]))
        self.check()

    def fork(self):
        if not self.want:
            return
        ids = list(self.want)
        parent = ids[int(self.rng.integers(0, len(ids)))]
        n = len(self.want[parent])
        pos = -1 if self.rng.random() < 0.5 else int(self.rng.integers(0, n + 1))
        child = self.next_id
        try:
            self.kv.fork_sequence(parent, child, pos)
        except RuntimeError:
            return                      # no page for the copy, too many sequences, or below a window's drop
        self.next_id += 1
        self.want[child] = list(self.want[parent][: n if pos < 0 else pos])
        if parent in self.window:
            self.window[child] = self.window[parent]

    def popn(self):
        ids = [s for s in self.want if self.want[s] and self.window.get(s, (0, 0))[0] == 0]
        if not ids:
            return
        sid = ids[int(self.rng.integers(0, len(ids)))]
        n = int(self.rng.integers(1, min(20, len(self.want[sid])) + 1))
        try:
            self.kv.popn(sid, n)
        except RuntimeError:
            return
        del self.want[sid][-n:]

    def remove(self):
        if not self.want:
            return
        ids = list(self.want)
        sid = ids[int(self.rng.integers(0, len(ids)))]
        self.kv.remove_sequence(sid)
        del self.want[sid]
        self.window.pop(sid, None)


@pytest.mark.parametrize("seed", range(6))
def test_random_operations_keep_every_history_readable(seed):
    sh = Shadow(num_pages=48 if seed % 2 else 200, max_seqs=10, seed=seed)
    ops = [sh.add, sh.forward, sh.forward, sh.forward, sh.tree, sh.fork, sh.fork, sh.popn, sh.remove]
    for _ in range(400):
        if len(sh.want) >= 10:
            sh.remove()
        ops[int(sh.rng.integers(0, len(ops)))]()
    sh.forward()
    for sid in list(sh.want):
        sh.kv.remove_sequence(sid)
    assert sh.kv.num_available_pages() == sh.num_pages
