"""Compile-and-tune with the reference's interface (yan/jit_kernels/tuner.py:8-80).

`compile_and_tune(name, keys, space, includes, arg_defs, template, args)` builds one kernel per
entry of `space` (each a dict of extra template keys), drops candidates whose launch returns a
non-zero code, times the rest and memoises the winner per (name, keys).  Changes for B200:
the L2 flush before timing covers twice the device's L2 (the reference's 128 MB, tuner.py:56, is
about the size of B200's L2), and winners are also persisted to a JSON file next to the kernel
cache so a new process does not re-time a known problem.
"""
from __future__ import annotations

import copy
import json
import os
from typing import Any, Dict

import torch

from ..jit import Runtime, build, cpp_format, generate
from ..jit.compiler import get_cache_dir
from ..utils import l2_flush_bytes


class JITTuner:
    def __init__(self) -> None:
        self.tuned: Dict[Any, Runtime] = {}

    @staticmethod
    def _store_path() -> str:
        return os.path.join(get_cache_dir(), "tuned.json")

    def _load_choice(self, key: str):
        try:
            with open(self._store_path(), "r") as f:
                return json.load(f).get(key)
        except (OSError, ValueError):
            return None

    def _save_choice(self, key: str, tuned_keys: dict) -> None:
        path = self._store_path()
        try:
            os.makedirs(os.path.dirname(path), exist_ok=True)
            data = {}
            if os.path.exists(path):
                with open(path, "r") as f:
                    data = json.load(f)
            data[key] = tuned_keys
            tmp = f"{path}.{os.getpid()}.tmp"
            with open(tmp, "w") as f:
                json.dump(data, f, indent=1, sort_keys=True)
            os.replace(tmp, path)
        except (OSError, ValueError):
            pass

    # ---- the four steps of compile_and_tune ----

    @staticmethod
    def _build_candidates(name, keys, space, includes, arg_defs, template):
        """One compiled Runtime per entry of the space (a build that fails raises)."""
        built = []
        for extra in space:
            assert isinstance(extra, dict), "every entry of the tuning space is a dict of template keys"
            merged = {**copy.deepcopy(keys), **extra}
            built.append((build(name, arg_defs, generate(includes, arg_defs, cpp_format(template, merged))), extra))
        return built

    @staticmethod
    def _is_legal(runtime: Runtime, args: tuple) -> int:
        """Launches once; the kernel's own return code says whether the configuration can run (0 = yes)."""
        return runtime(*args)

    @staticmethod
    def _time(runtime: Runtime, args: tuple, scrub: torch.Tensor, launches: int = 20) -> float:
        """Milliseconds for `launches` back-to-back launches after the L2 has been overwritten."""
        first, last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        scrub.zero_()
        first.record()
        for _ in range(launches):
            code = runtime(*args)
            assert code == 0, f"a launch that was legal a moment ago returned {code}"
        last.record()
        last.synchronize()
        return first.elapsed_time(last)

    def compile_and_tune(self, name: str, keys: Dict[str, Any], space: tuple, includes: tuple, arg_defs: tuple,
                         template: str, args: tuple) -> Runtime:
        """Signature and meaning of yan/jit_kernels/tuner.py:12: returns the fastest legal kernel of `space` for
        (name, keys), remembered for the life of the process and, across processes, in tuned.json.
        The space and the template must not change for a given (name, keys), and the kernel must be repeatable: it
        is launched many times while it is timed."""
        verbose = bool(os.getenv("YAN_JIT_DEBUG"))
        keys = dict(sorted(keys.items()))
        memo_key = (name, f"{keys}")
        if memo_key in self.tuned:
            if verbose:
                print(f"[tuner] {name} {keys}: already tuned in this process")
            return self.tuned[memo_key]
        assert args is not None, "tuning needs one set of launch arguments"
        candidates_space = tuple(space) if len(space) > 0 else ({},)
        contest = len(candidates_space) > 1

        device = torch.cuda.get_device_name() if torch.cuda.is_available() else "nodevice"
        store_key = f"{name}|{keys}|{device}"
        if contest:
            remembered = self._load_choice(store_key)
            if remembered is not None and remembered in list(candidates_space):
                if verbose:
                    print(f"[tuner] {name} {keys}: tuned.json holds {remembered}")
                candidates_space, contest = (remembered,), False

        built = self._build_candidates(name, keys, candidates_space, includes, arg_defs, template)
        if not contest:
            winner, winner_keys, winner_ms = built[0][0], built[0][1], 0.0
        else:
            scrub = torch.empty(l2_flush_bytes() // 4, dtype=torch.int, device="cuda")
            winner, winner_keys, winner_ms = None, None, None
            for runtime, extra in built:
                code = self._is_legal(runtime, args)
                if code != 0:
                    if verbose:
                        print(f"[tuner] {name} {keys} + {extra}: refused with return code {code}, skipped")
                    continue
                ms = self._time(runtime, args, scrub)
                if verbose:
                    print(f"[tuner] {name} {keys} + {extra}: {ms:.3f} ms for 20 launches")
                if winner_ms is None or ms < winner_ms:
                    winner, winner_keys, winner_ms = runtime, extra, ms
            assert winner is not None, f"no configuration of {name} with keys {keys} could be launched"
            self._save_choice(store_key, winner_keys)
        if verbose or os.getenv("YAN_PRINT_AUTOTUNE"):
            print(f"[tuner] {name} {keys}: chose {winner_keys} ({winner_ms:.3f} ms)")
        self.tuned[memo_key] = winner
        return winner


jit_tuner = JITTuner()
