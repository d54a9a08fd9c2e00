"""Progress bar that fills from right to left (used for the backward sweep)."""

from tqdm.auto import tqdm


class RtlTqdm(tqdm):
    @staticmethod
    def format_meter(*args, **kwargs):
        line = tqdm.format_meter(*args, **kwargs)
        start, end = line.find("|"), line.rfind("|")
        if 0 <= start < end:
            bar = line[start + 1 : end]
            line = line[: start + 1] + bar[::-1] + line[end:]
        return line
