"""Hierarchical state machine substrate (reference: crates/hfsm/src/lib.rs — UML-statechart
dispatch: an unhandled event bubbles to the superstate; a transition exits bottom-up from the
active leaf to, and not including, the least common ancestor of source and target, then enters
top-down to the target; entry / exit actions cannot move the machine; events posted while an
event is being handled are processed after it, run to completion, which is what drives streaming
by a state posting itself a reminder).

A machine is any object with ``dispatch(state, event) -> Handled | Unhandled | Tran(target) |
Super(state)``, ``parent(state) -> state | None`` and optional ``on_entry(state)`` /
``on_exit(state)``."""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass
from typing import Any, Deque, List, Optional


class _Handled:
    def __repr__(self):
        return "Handled"


class _Unhandled:
    def __repr__(self):
        return "Unhandled"


Handled = _Handled()
Unhandled = _Unhandled()


@dataclass(frozen=True)
class Tran:
    target: Any


@dataclass(frozen=True)
class Super:
    state: Any


class Hsm:
    def __init__(self, machine, initial):
        self.machine = machine
        self.state = initial
        self._queue: Deque = deque()
        self._running = False

    # ---- structure
    def _path_to_root(self, s) -> List:
        out = [s]
        while True:
            p = self.machine.parent(out[-1])
            if p is None:
                return out
            out.append(p)

    def _lca(self, a, b):
        anc = self._path_to_root(a)
        return next((c for c in self._path_to_root(b) if c in anc), None)

    def in_state(self, s) -> bool:
        """True when ``s`` is the active state or one of its ancestors."""
        return s in self._path_to_root(self.state)

    # ---- driving
    def init(self) -> None:
        """Enter the initial configuration top-down, then drain whatever the entries posted."""
        for s in reversed(self._path_to_root(self.state)):
            self._call("on_entry", s)
        self.run()

    def post(self, event) -> None:
        self._queue.append(event)

    def run(self) -> None:
        if self._running:                 # non-reentrant: a handler that calls run() only enqueues
            return
        self._running = True
        try:
            while self._queue:
                self._step(self._queue.popleft())
        finally:
            self._running = False

    def send(self, event) -> None:
        self.post(event)
        self.run()

    def _call(self, name: str, s) -> None:
        fn = getattr(self.machine, name, None)
        if fn is not None:
            fn(s)

    def _step(self, event) -> None:
        source = self.state
        while True:
            d = self.machine.dispatch(source, event)
            if d is Handled:
                return
            if isinstance(d, Tran):
                break
            source = d.state if isinstance(d, Super) else self.machine.parent(source)
            if source is None:
                return                    # reached the top unhandled: ignored (the UML default)
        target = d.target
        lca = self._lca(source, target)
        s: Optional[Any] = self.state
        while s is not None and s != lca:
            self._call("on_exit", s)
            s = self.machine.parent(s)
        path = []
        t = target
        while t is not None and t != lca:
            path.append(t)
            t = self.machine.parent(t)
        for st in reversed(path):
            self._call("on_entry", st)
        self.state = target
