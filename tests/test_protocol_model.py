"""Model test of the Fabric's slot protocol with the host instance of the device scheduler.

Producers (attention ranks) bump a per-slot sequence word; Lanes poll the words, enqueue what is ahead of
the slot's completed sequence, get a lease from the scheduler, serve and release. Hypothesis drives
arbitrary interleavings of publishes, polls and completions; the invariants are the ones the device code
relies on: every published sequence is served exactly once and in order per slot, a slot is never served
by two Lanes at once, a Lane never holds two slots, and nothing is served that was not published.
"""
from hypothesis import given, settings
from hypothesis import strategies as st

from crosspool_b200.native import runtime as rt

N_SLOTS, N_LANES = 4, 2


class Model:
    def __init__(self, policy):
        self.s = rt.LaneScheduler(N_SLOTS, N_LANES, policy, seed=7)
        self.published = [0] * N_SLOTS      # sequence word of every slot
        self.done = [0] * N_SLOTS           # completed sequence as the Lanes see it
        self.queued = [False] * N_SLOTS
        self.running = {}                   # lane -> (slot, sequence, lease)
        self.served = [[] for _ in range(N_SLOTS)]

    def publish(self, slot):
        # an attention rank publishes its next invocation only after the previous one completed
        if self.published[slot] == self.done[slot]:
            self.published[slot] += 1

    def poll(self):
        """One lane_wait pass: enqueue slots that are ahead, then try to lease a Lane."""
        for i in range(N_SLOTS):
            ahead = self.published[i] - self.done[i]
            busy = any(v[0] == i for v in self.running.values())
            if ahead > 0 and not self.queued[i] and not busy:
                assert self.s.enqueue(i, self.done[i] + ahead, deadline=100 + i)
                self.queued[i] = True
        d = self.s.try_schedule()
        if d is not None:
            slot, lane, lease = d
            assert lane not in self.running, "a Lane was leased twice"
            assert all(v[0] != slot for v in self.running.values()), "a slot is being served by two Lanes"
            assert self.queued[slot]
            self.queued[slot] = False
            self.running[lane] = (slot, self.published[slot], lease)

    def complete(self, lane):
        if lane not in self.running:
            return
        slot, seq, lease = self.running.pop(lane)
        assert self.s.release(slot, lease)
        assert seq == self.done[slot] + 1, "served out of order"
        self.done[slot] = seq
        self.served[slot].append(seq)


ops = st.lists(st.one_of(st.tuples(st.just("publish"), st.integers(0, N_SLOTS - 1)),
                         st.tuples(st.just("poll"), st.just(0)),
                         st.tuples(st.just("complete"), st.integers(0, N_LANES - 1))), min_size=1, max_size=200)


@settings(max_examples=150, deadline=None)
@given(ops, st.sampled_from([rt.POLICY_FIFO, rt.POLICY_RANDOM, rt.POLICY_SLO]))
def test_every_publication_is_served_once_in_order_under_any_interleaving(trace, policy):
    m = Model(policy)
    for op, arg in trace:
        getattr(m, op)(*(() if op == "poll" else (arg,)))
    # drain: keep polling and completing until nothing is outstanding
    for _ in range(4 * N_SLOTS + 8):
        m.poll()
        for lane in range(N_LANES):
            m.complete(lane)
    for i in range(N_SLOTS):
        assert m.served[i] == list(range(1, m.published[i] + 1))
        assert m.done[i] == m.published[i]
    m.s.close()
