"""``Progbar``: text progress bar (keras/src/utils/progbar.py)."""

import math
import os
import sys
import time

from keras_b200.core.export_registry import keras_export
from keras_b200.utils import io_utils


@keras_export("keras.utils.Progbar")
class Progbar:
    def __init__(self, target, width=20, verbose=1, interval=0.05, stateful_metrics=None, unit_name="step"):
        self.target = target
        self.width = width
        self.verbose = verbose
        self.interval = interval
        self.unit_name = unit_name
        self.stateful_metrics = set(stateful_metrics) if stateful_metrics else set()
        self._dynamic_display = (hasattr(sys.stdout, "isatty") and sys.stdout.isatty()) or "ipykernel" in sys.modules or "posix" in sys.modules or "PYCHARM_HOSTED" in os.environ
        self._seen_so_far = 0
        self._values = {}
        self._values_order = []
        self._start = time.time()
        self._last_update = 0
        self._time_at_epoch_start = self._start
        self._time_after_first_step = None
        self._prev_total_width = 0

    def update(self, current, values=None, finalize=None):
        if finalize is None:
            finalize = False if self.target is None else current >= self.target
        values = values or []
        for k, v in values:
            if k not in self._values_order:
                self._values_order.append(k)
            if k not in self.stateful_metrics:
                value_base = max(current - self._seen_so_far, 1)
                if k not in self._values:
                    self._values[k] = [v * value_base, value_base]
                else:
                    self._values[k][0] += v * value_base
                    self._values[k][1] += value_base
            else:
                self._values[k] = [v, 1]
        self._seen_so_far = current
        message = ""
        special_char_len = 0
        now = time.time()
        time_per_unit = self._estimate_step_duration(current, now)
        if self.verbose == 1:
            if now - self._last_update < self.interval and not finalize:
                return
            if self._dynamic_display:
                message += "\b" * self._prev_total_width
                message += "\r"
            else:
                message += "\n"
            if self.target is not None:
                numdigits = int(math.log10(self.target)) + 1 if self.target > 0 else 1
                bar = ("%" + str(numdigits) + "d/%d") % (current, self.target)
                bar = f"\x1b[1m{bar}\x1b[0m "
                special_char_len += 8
                prog = float(current) / self.target if self.target else 1.0
                prog_width = int(self.width * prog)
                if prog_width > 0:
                    bar += "\33[32m" + "━" * prog_width + "\x1b[0m"
                    special_char_len += 9
                bar += "\33[37m" + "━" * (self.width - prog_width) + "\x1b[0m"
                special_char_len += 9
            else:
                bar = "%7d/Unknown" % current
            message += bar
            if self.target is not None and not finalize:
                eta = time_per_unit * (self.target - current)
                if eta > 3600:
                    eta_format = "%d:%02d:%02d" % (eta // 3600, (eta % 3600) // 60, eta % 60)
                elif eta > 60:
                    eta_format = "%d:%02d" % (eta // 60, eta % 60)
                else:
                    eta_format = "%ds" % eta
                info = f" \x1b[1m{eta_format}\x1b[0m"
            else:
                info = f" \x1b[1m{now - self._start:.0f}s\x1b[0m"
            special_char_len += 8
            info += self._format_time(time_per_unit, self.unit_name)
            for k in self._values_order:
                info += f" - {k}:"
                if isinstance(self._values[k], list):
                    avg = float(self._values[k][0]) / max(1, self._values[k][1])
                    info += f" {avg:.4f}" if abs(avg) > 1e-3 else f" {avg:.4e}"
                else:
                    info += f" {self._values[k]}"
            message += info
            total_width = len(bar) + len(info) - special_char_len
            if self._prev_total_width > total_width:
                message += " " * (self._prev_total_width - total_width)
            if finalize:
                message += "\n"
            io_utils.print_msg(message, line_break=False)
            self._prev_total_width = total_width
        elif self.verbose == 2:
            if finalize:
                numdigits = int(math.log10(self.target)) + 1 if self.target else 1
                count = ("%" + str(numdigits) + "d/%d") % (current, self.target or current)
                info = f"{count} - {now - self._start:.0f}s"
                info += " -" + self._format_time(time_per_unit, self.unit_name)
                for k in self._values_order:
                    info += f" - {k}:"
                    avg = float(self._values[k][0]) / max(1, self._values[k][1])
                    info += f" {avg:.4f}" if avg > 1e-3 else f" {avg:.4e}"
                info += "\n"
                io_utils.print_msg(info, line_break=False)
        self._last_update = now

    def add(self, n, values=None):
        self.update(self._seen_so_far + n, values)

    def _format_time(self, time_per_unit, unit_name):
        if time_per_unit >= 1 or time_per_unit == 0:
            return f" {time_per_unit:.0f}s/{unit_name}"
        if time_per_unit >= 1e-3:
            return f" {time_per_unit * 1e3:.0f}ms/{unit_name}"
        return f" {time_per_unit * 1e6:.0f}us/{unit_name}"

    def _estimate_step_duration(self, current, now):
        if current:
            if self._time_after_first_step is not None and current > 1:
                return (now - self._time_after_first_step) / (current - 1)
            if current == 1:
                self._time_after_first_step = now
            return (now - self._start) / current
        return 0
