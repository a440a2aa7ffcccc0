"""One-line training progress display with a 20-step rolling average of step time, written with a carriage return
(serenitymojo/training/progress_display.mojo: line format and the H:MM:SS rendering)."""
from __future__ import annotations

import sys
import time
from collections import deque


def format_hms(seconds: float) -> str:
    s = int(max(0, seconds))
    return f"{s // 3600}:{(s % 3600) // 60:02d}:{s % 60:02d}"


class ProgressDisplay:
    def __init__(self, name: str, total_steps: int, total_epochs: int = 1, window: int = 20, stream=None, clock=time.monotonic):
        self.name, self.total, self.epochs = name, total_steps, total_epochs
        self.times = deque(maxlen=window)
        self.stream = stream if stream is not None else sys.stdout
        self.clock = clock
        self.t0 = clock()
        self.last = self.t0

    def line(self, step: int, epoch: int, loss: float, grad_norm: float) -> str:
        now = self.clock()
        self.times.append(now - self.last)
        self.last = now
        avg = sum(self.times) / len(self.times)
        eta = avg * max(0, self.total - step)
        return (f"[{self.name}] step {step}/{self.total} | epoch {epoch}/{self.epochs} | loss {loss:.4f} | "
                f"grad_norm {grad_norm:.4f} | {avg:.1f}s/step | elapsed {format_hms(now - self.t0)} | ETA {format_hms(eta)}")

    def update(self, step: int, epoch: int, loss: float, grad_norm: float) -> str:
        s = self.line(step, epoch, loss, grad_norm)
        self.stream.write("\r" + s)
        self.stream.flush()
        return s

    def finish(self) -> None:
        self.stream.write("\n")
        self.stream.flush()
