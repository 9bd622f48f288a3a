"""``QuantizationReport``: which layers ``Model.quantize`` quantized, skipped (and why) or failed on
(keras/src/quantizers/report.py)."""

from keras_b200.core.export_registry import keras_export


@keras_export("keras.quantizers.QuantizationReport")
class QuantizationReport:
    SKIP_NO_SUPPORT = "no quantize support"
    SKIP_FILTERED = "filtered out"
    SKIP_ALREADY_QUANTIZED = "already quantized"
    SKIP_OUTSIDE_STRUCTURE = "outside quantization structure"

    def __init__(self, mode=None):
        self.mode = mode
        self.quantized, self.skipped, self.errors = [], [], []

    def add_quantized(self, path, mode, scheme):
        self.quantized.append((path, mode, scheme))

    def add_skipped(self, path, reason):
        self.skipped.append((path, reason))

    def add_error(self, path, error):
        self.errors.append((path, str(error)))

    num_quantized = property(lambda self: len(self.quantized))
    num_skipped = property(lambda self: len(self.skipped))
    num_errors = property(lambda self: len(self.errors))

    def skipped_by_reason(self, reason):
        return [path for path, r in self.skipped if r == reason]

    def summary_warning(self, max_examples=5):
        unsupported = self.skipped_by_reason(self.SKIP_NO_SUPPORT)
        if not unsupported and not self.errors:
            return None

        def examples(paths):
            text = ", ".join(repr(p) for p in paths[:max_examples])
            return text + (", ..." if len(paths) > max_examples else "")

        parts = []
        if unsupported:
            parts.append(f"{len(unsupported)} layer(s) were skipped because they do not support quantization (e.g. {examples(unsupported)}).")
        if self.errors:
            parts.append(f"{len(self.errors)} layer(s) reported errors (e.g. {examples([p for p, _ in self.errors])}).")
        parts.append(f"Quantized {self.num_quantized} layer(s) in mode '{self.mode}'. Call `model.quantization_summary()` or inspect the returned `QuantizationReport` for details.")
        return "`model.quantize()`: " + " ".join(parts)

    def render(self):
        lines = [f"Quantization report (mode='{self.mode}')", "=" * 65, f"Quantized {self.num_quantized} layer(s):"]
        lines += [f"  - {p} ({m}): {s}" for p, m, s in self.quantized] or ["  (none)"]
        lines.append(f"Skipped {self.num_skipped} layer(s):")
        lines += [f"  - {p}: {r}" for p, r in self.skipped] or ["  (none)"]
        if self.errors:
            lines.append(f"Errors on {self.num_errors} layer(s):")
            lines += [f"  - {p}: {m}" for p, m in self.errors]
        return "\n".join(lines)

    __str__ = render

    def __repr__(self):
        return f"QuantizationReport(mode={self.mode!r}, quantized={self.num_quantized}, skipped={self.num_skipped}, errors={self.num_errors})"

    @classmethod
    def from_model(cls, model):
        report = getattr(model, "_quantization_report", None)
        return report if report is not None else cls(mode=None)
