"""Prefix parking on CPU tensors: save/restore/rewind through ring checkpoints, resume selection, eviction."""
import torch

from naivert_b200.runtime.prefix_store import ParkedPrefix, PrefixStore, park_name, select_resume


def _store(budget=1 << 20):
    full = [torch.zeros(64, 4), torch.zeros(64, 2)]
    rings = [torch.zeros(8, 4)]
    return full, rings, PrefixStore(full, rings, budget)


def test_save_restore_roundtrip_and_rewind():
    full, rings, st = _store()
    for t in full:
        t.copy_(torch.arange(t.numel(), dtype=torch.float32).reshape(t.shape))
    rings[0].fill_(1.0)
    ck = st.make_checkpoint(10)                  # ring state at prompt end, kept by the session
    rings[0].fill_(2.0)
    st.save("a", list(range(30)), 29, checkpoints=[ck])
    saved = [t.clone() for t in full]
    for t in full:
        t.zero_()
    rings[0].zero_()
    ch = select_resume(st.entries, list(range(30)) + [99, 98], "a")
    assert ch.position == 29 and ch.checkpoint is None
    assert st.restore(ch) == 29
    assert torch.equal(full[0][:29], saved[0][:29]) and float(full[0][29:].abs().sum()) == 0
    assert float(rings[0][0, 0]) == 2.0
    # a branch that shares only 20 tokens rewinds to the ring checkpoint at 10
    ch = select_resume(st.entries, list(range(20)) + [7, 7, 7], "a", min_gain=4)
    assert ch.position == 10 and ch.checkpoint == 0
    st.restore(ch)
    assert float(rings[0][0, 0]) == 1.0


def test_branch_then_rewind_never_takes_the_other_branch_rings():
    """Conversation A is parked under its session key; a branch of the same session is parked as ``key#1`` with its
    own prompt-end checkpoint.  A later rewind inside A must get rings taken while A was in the caches."""
    full, rings, st = _store()
    a_prompt = list(range(100, 140))                                    # 40 tokens
    rings[0].fill_(1.0)
    ck_a = st.make_checkpoint(39)
    rings[0].fill_(2.0)
    a_seq = a_prompt + list(range(500, 520))
    st.save(park_name(st.entries, "S", a_seq), a_seq, 59, checkpoints=[ck_a])
    # a branch that shares 20 tokens with A, 120 tokens long, same session id
    b_seq = a_prompt[:20] + list(range(900, 1000))
    rings[0].fill_(7.0)
    ck_b = st.make_checkpoint(119)
    rings[0].fill_(8.0)
    name_b = park_name(st.entries, "S", b_seq)
    assert name_b == "S#1"
    st.save(name_b, b_seq, 119, checkpoints=[ck_b])
    # rewind inside A: shares 50 tokens with A (beyond A's prompt end at 39), 20 with the branch
    req = a_seq[:50] + [1, 2, 3]
    ch = select_resume(st.entries, req, "S", min_gain=4)
    assert ch.key == "S" and ch.position == 39 and ch.checkpoint is not None
    st.restore(ch)
    assert float(rings[0][0, 0]) == 1.0                                 # A's rings at its prompt end, not the branch's
    # no entry carries a checkpoint beyond its own tokens
    for e in st.entries.values():
        assert all(c.position <= e.position for c in e.checkpoints)
    # replacing A by a sequence that diverges at 30 drops A's checkpoint at 39
    st.save("S", a_seq[:30] + [4] * 40, 69)
    assert all(c.position <= 30 for c in st.entries["S"].checkpoints)


def test_selection_prefers_longest_then_own_key():
    e1 = ParkedPrefix("s1", list(range(100)), 99, [], [])
    e2 = ParkedPrefix("s2", list(range(100)), 99, [], [])
    e3 = ParkedPrefix("s3", list(range(50)), 49, [], [])
    entries = {"s1": e1, "s2": e2, "s3": e3}
    assert select_resume(entries, list(range(120)), "s2").key == "s2"
    assert select_resume(entries, list(range(60)) + [1], "s3").key == "s3"      # s1/s2 parks lie beyond the match
    assert select_resume(entries, [5, 6, 7], None) is None
    assert select_resume(entries, list(range(100)), "s1") is None or select_resume(entries, list(range(100)), "s1").position <= 99


def test_park_name_branches():
    entries = {"k": ParkedPrefix("k", list(range(40)), 39, [], [])}
    assert park_name(entries, "k", list(range(60))) == "k"
    assert park_name(entries, "k", list(range(20)) + [0] * 30) == "k#1"
    assert park_name(entries, None, [1, 2]) == "anon"


def test_eviction_lru_to_budget():
    full, rings, st = _store(budget=3000)
    st.save("a", list(range(40)), 39)
    st.save("b", list(range(40)), 39)
    st.entries["a"].last_used += 100            # a is fresher than b
    st.save("c", list(range(40)), 39)
    assert "c" in st.entries and st.bytes() <= 3000 and "b" not in st.entries


def test_prefill_policy_and_segment_stats():
    from naivert_b200.runtime.session_engine import prefill_estimate, prefill_path, segment_stats
    assert prefill_estimate(0, "replay") == 0
    assert prefill_path(100, "cost", native_ready=True) == "native" if prefill_estimate(100, "native") < prefill_estimate(100, "replay") else "replay"
    assert prefill_path(10, "cost", native_ready=True) == "replay"
    assert prefill_path(100000, "cost", native_ready=True) == "native"
    assert prefill_path(100000, "cost", native_ready=False) == "replay" and prefill_path(5, "native", native_ready=True) == "native"
    toks = [1, 2, 9, 4, 5, 6, 7, 8]
    st = segment_stats(toks, [3, 3, 2], [1000, 4000, 8000], think_end=9, accepted=[2, 2, 1])
    assert st["think"]["tokens"] == 3 and st["answer"]["tokens"] == 5 and st["total"]["rounds"] == 2
    assert st["total"]["device_ms"] == 0.007 and st["answer"]["device_tok_s"] > 0


def test_align_prompt_keeps_sampled_ids_of_a_parked_history():
    """The sampler wrote "ab" as two ids; the encoder would write one.  The canonical ids of the follow-up prompt
    therefore diverge from the parked ids inside the history, but the decoded text still extends it: the parked ids
    are kept and only the new text is encoded."""
    from types import SimpleNamespace
    from naivert_b200.runtime.session_engine import SessionEngine

    class Tok:                               # ids 0..25 = letters, 26 = the merged pair "ab"
        def decode(self, ids):
            return "".join("ab" if i == 26 else chr(97 + i) for i in ids)

        def encode(self, text):
            out, i = [], 0
            while i < len(text):
                if text.startswith("ab", i):
                    out.append(26); i += 2
                else:
                    out.append(ord(text[i]) - 97); i += 1
            return out

    se = SessionEngine.__new__(SessionEngine)
    full, rings, st = _store()
    se.store, se.tokenizer = st, Tok()
    se.engine = SimpleNamespace(spec=SimpleNamespace(vocab=27))
    sampled = [2, 3] * 10 + [0, 1] + [4] * 10           # "cd"*10 + "a","b" (sampled split) + "e"*10
    st.save("S", sampled, 30)                             # parks 30 ids = text "cd"*10 + "ab" + "e"*8
    text = Tok().decode(sampled) + "xyz"
    canonical = Tok().encode(text)
    assert canonical[:22] != sampled[:22]                 # the encoder merges "ab"
    assert select_resume(st.entries, canonical, "S") is None or select_resume(st.entries, canonical, "S").position < 30
    aligned = se.align_prompt(canonical, "S", text=text)
    assert aligned[:30] == sampled[:30] and Tok().decode(aligned) == text
    assert select_resume(st.entries, aligned, "S").position == 30
    # ids already match: unchanged; no tokenizer or no text: unchanged
    assert se.align_prompt(sampled + [5], "S", text=Tok().decode(sampled + [5])) == sampled + [5]
    assert se.align_prompt(canonical, "S") == canonical
    se.tokenizer = None
    assert se.align_prompt(canonical, "S", text=text) == canonical


def test_best_prefix_match_is_the_closest_parked_entry():
    from naivert_b200.runtime.prefix_store import best_prefix_match
    entries = {"a": ParkedPrefix("a", list(range(100)), 99, [], []),
               "b": ParkedPrefix("b", list(range(40)) + [7] * 60, 99, [], []),
               "c": ParkedPrefix("c", list(range(100)), 30, [], [])}          # only 30 positions are parked
    assert best_prefix_match(entries, list(range(60)) + [1, 2]) == ("a", 60)
    assert best_prefix_match(entries, list(range(40)) + [7, 7, 9]) == ("b", 42)
    assert best_prefix_match({"c": entries["c"]}, list(range(100))) == ("c", 30)
    assert best_prefix_match({}, [1, 2]) is None and best_prefix_match(entries, [5])[1] == 0
