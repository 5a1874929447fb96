"""Record how the REFERENCE's radix prefix cache drives a block manager, as a replayable fixture.

    python tests/golden/make_block_trace.py /path/to/LLM-CompileForge

The reference's Python ``RadixCache`` (python_runtime/engine/cache/radix_cache.py, imported from the checkout, never
copied) runs over the oracle's block-manager restatement through a recording proxy while a small serving loop plays:
requests arrive with prompts that share prefixes, take their cached blocks (``match_prefix`` -> ``assign_cached_blocks`` +
``ensure_blocks``) or allocate, decode a few tokens, finish (``insert`` into the tree, ``free``), and now and then the
cache evicts.  Every block-manager call - the engine's and the ones ``RadixCache`` makes itself (``increment_ref_count``,
``free_block``) - is written to ``block_manager_trace.json`` with its result and the free-block count after it.
tests/test_block_manager.py replays the calls on the C++ manager."""

from __future__ import annotations

import json
import os
import random
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))


class Recorder:
    def __init__(self, inner, log):
        self._inner, self._log = inner, log
        self.block_size = inner.block_size

    def __getattr__(self, name):
        fn = getattr(self._inner, name)

        def call(*args):
            try:
                res = fn(*args)
                out = {"ok": res if not isinstance(res, float) else round(res, 9)}
            except Exception as e:  # noqa: BLE001
                out = {"raises": type(e).__name__}
            self._log.append({"op": name, "args": [list(a) if isinstance(a, (list, tuple)) else a for a in args], **out,
                              "free": self._inner.num_free_blocks()})
            if "raises" in out:
                raise
            return res

        return call


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    sys.path.insert(0, REPO)
    from python_runtime.engine.cache.radix_cache import RadixCache

    from oracle.block_manager_port import BlockManagerPort

    traces = []
    for seed, (nb, bs) in enumerate([(26, 4), (160, 16)]):
        rng = random.Random(100 + seed)
        log: list[dict] = []
        bm = Recorder(BlockManagerPort(nb, bs), log)
        radix = RadixCache(bm)
        system = [rng.randrange(1000) for _ in range(3 * bs + 1)]
        live: dict[str, list[int]] = {}
        for step in range(120):
            act = rng.random()
            if act < 0.45 and len(live) < 6:
                rid = f"req{step}"
                share = rng.choice([0, bs, 2 * bs, len(system)])
                tokens = system[:share] + [rng.randrange(1000) for _ in range(rng.randint(1, 3 * bs))]
                cached, matched = radix.match_prefix(tokens)
                try:
                    if cached:
                        bm.assign_cached_blocks(rid, cached)
                        bm.ensure_blocks(rid, len(tokens))
                    else:
                        bm.allocate(rid, len(tokens))
                    live[rid] = tokens
                except Exception:  # noqa: BLE001  (pool exhausted: the request is dropped, its cached blocks released)
                    bm.free(rid)
            elif act < 0.75 and live:
                rid = rng.choice(list(live))
                live[rid].append(rng.randrange(1000))
                try:
                    bm.ensure_blocks(rid, len(live[rid]) + 1)
                except Exception:  # noqa: BLE001
                    pass
            elif act < 0.92 and live:
                rid = rng.choice(list(live))
                radix.insert(live[rid], bm.get_blocks(rid))
                bm.free(rid)
                del live[rid]
            else:
                # the engine drops its hold on some cached sequences, then asks for room
                stack = list(radix.root.children.values())
                while stack:
                    node = stack.pop()
                    if rng.random() < 0.5:
                        node.ref_count = 0
                    stack.extend(node.children.values())
                radix.evict(rng.randint(1, 6))
            bm.num_free_blocks()
        for rid in list(live):
            bm.get_blocks(rid)
        traces.append({"num_blocks": nb, "block_size": bs, "calls": log})
    with open(os.path.join(HERE, "block_manager_trace.json"), "w") as f:
        json.dump(traces, f, separators=(",", ":"))
    print(sum(len(t["calls"]) for t in traces), "calls recorded")


if __name__ == "__main__":
    sys.path.insert(0, REPO)
    from oracle.build_ref import reference_root  # argument, $SFB_REFERENCE_ROOT, or ../reference beside this repository

    main(reference_root(sys.argv[1] if len(sys.argv) > 1 and not sys.argv[1].startswith("--") else None))
