"""Tiny CSV appender that can be disabled on non-zero ranks."""

from __future__ import annotations

import csv
import os


class CSVWriter:
    def __init__(self, path: str, columns, enabled: bool = True):
        self.enabled = enabled
        self.file = None
        if enabled:
            os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
            self.file = open(path, "w", newline="")
            self.writer = csv.writer(self.file)
            self.writer.writerow(list(columns))

    def writerow(self, *values):
        if self.enabled:
            self.writer.writerow(list(values))
            self.file.flush()

    def close(self):
        if self.file is not None:
            self.file.close()
            self.file = None
