"""Build-every-candidate auto-tuner.

Contract of the reference tuner (fray/jit_kernels/tuner.py:12-78): for one
``(name, keys)`` signature, generate and build every point of ``space``, run each once
to weed out candidates whose ``launch`` reports a non-zero code, flush L2, time 20
back-to-back launches between CUDA events and memoise the fastest ``Runtime``.

Additions: ``keys`` may carry entries the template does not mention (a shape class, the
causal flag) so that one op can be tuned per workload class instead of once per head
dim; the winner is also written to ``tuned.json`` beside the kernel cache and reused by
later processes on the same device model; ``FRAY_ATTN_FORCE`` style overrides are handled
by the op, which then passes a one-point space.
"""
import copy
import json
import os
from typing import Any, Dict

import torch

from ..jit import Runtime, build, cpp_format, generate
from ..jit.compiler import get_default_user_dir, get_fray_version, put


def _debug() -> bool:
    return bool(os.getenv("FRAY_JIT_DEBUG"))


class JITTuner:
    def __init__(self) -> None:
        self.tuned: Dict[Any, Runtime] = {}
        self.tuned_keys: Dict[Any, Dict[str, Any]] = {}

    # ------------------------------------------------------------------ persistence
    @staticmethod
    def _db_path() -> str:
        return os.path.join(get_default_user_dir(), "tuned.json")

    def _db_key(self, signature) -> str:
        device = torch.cuda.get_device_name() if torch.cuda.is_available() else "nodevice"
        return f"{device}|{get_fray_version()}|{signature[0]}|{signature[1]}"

    def _db_load(self) -> Dict[str, Any]:
        try:
            with open(self._db_path(), "r") as f:
                return json.load(f)
        except (OSError, ValueError):
            return {}

    def _db_store(self, signature, tuned_keys: Dict[str, Any]) -> None:
        if os.getenv("FRAY_DISABLE_TUNE_DB"):
            return
        db = self._db_load()
        db[self._db_key(signature)] = tuned_keys
        try:
            put(self._db_path(), json.dumps(db, indent=1, sort_keys=True))
        except OSError:
            pass

    # ------------------------------------------------------------------ timing
    @staticmethod
    def time_candidate(runtime: Runtime, args: tuple, launches: int = 20) -> float:
        """Milliseconds for ``launches`` back-to-back calls after an L2 flush (reference: tuner.py:52-63).

        Differences from the reference: three untimed launches first (the first launch of a library pays
        module loading and the tensor-map encodings), and the best of three timed rounds, so that a
        candidate is not dropped for one slow round (causal shapes were seen to vary by 10 % from run to
        run on one box).
        """
        for _ in range(3):
            assert runtime(*args) == 0
        best = None
        for _ in range(3):
            start = torch.cuda.Event(enable_timing=True)
            end = torch.cuda.Event(enable_timing=True)
            torch.empty(int(256e6 // 4), dtype=torch.int, device="cuda").zero_()
            start.record()
            for _ in range(launches):
                assert runtime(*args) == 0
            end.record()
            end.synchronize()
            elapsed = start.elapsed_time(end)
            best = elapsed if best is None else min(best, elapsed)
        return best

    # ------------------------------------------------------------------ main entry
    def compile_and_tune(self, name: str, keys: Dict[str, Any], space: tuple, includes: tuple, arg_defs: tuple,
                         template: str, args: tuple, epilogue: str = "") -> Runtime:
        keys = {k: keys[k] for k in sorted(keys.keys())}
        signature = (name, f"{keys}")
        if signature in self.tuned:
            if _debug():
                print(f"Using cached JIT kernel {name} with keys {keys}")
            return self.tuned[signature]
        if _debug():
            print(f"Auto-tuning JIT kernel {name} with keys {keys}")
        assert args is not None
        space = (dict(),) if len(space) == 0 else tuple(space)

        def make(tuned_keys: Dict[str, Any]) -> Runtime:
            full_keys = copy.deepcopy(keys)
            full_keys.update(tuned_keys)
            code = generate(includes, arg_defs, cpp_format(template, full_keys), cpp_format(epilogue, full_keys))
            return build(name, arg_defs, code)  # an illegal build raises

        # A winner recorded by an earlier process on the same device model short-cuts the search.
        if len(space) > 1 and not os.getenv("FRAY_DISABLE_TUNE_DB"):
            remembered = self._db_load().get(self._db_key(signature))
            if remembered is not None and any(remembered == dict(p) for p in space):
                runtime = make(remembered)
                self.tuned[signature] = runtime
                self.tuned_keys[signature] = remembered
                return runtime

        kernels = [(make(tuned_keys), tuned_keys) for tuned_keys in space]

        best_runtime, best_time, best_keys = None, None, None
        for runtime, tuned_keys in kernels:
            if len(space) > 1:
                return_code = runtime(*args)
                if return_code != 0:
                    if _debug():
                        print(f"Illegal JIT kernel {name} with keys {keys} and tuned keys {tuned_keys}: "
                              f"error code {return_code}")
                    continue
                elapsed = self.time_candidate(runtime, args)
            else:
                elapsed = 0
            if best_time is None or elapsed < best_time:
                best_runtime, best_time, best_keys = runtime, elapsed, tuned_keys
            if _debug():
                print(f"Tuned JIT kernel {name} with keys {keys} and tuned keys {tuned_keys} has time {elapsed}")
        assert best_runtime is not None, f"Failed to tune JIT kernel {name} with keys {keys}"

        if _debug() or os.getenv("FRAY_PRINT_AUTOTUNE"):
            print(f"Best JIT kernel {name} with keys {keys} has tuned keys {best_keys} and time {best_time}")
        self.tuned[signature] = best_runtime
        self.tuned_keys[signature] = best_keys
        if len(space) > 1:
            self._db_store(signature, best_keys)
        return best_runtime


jit_tuner = JITTuner()
