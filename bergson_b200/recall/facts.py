"""Seeded synthetic people and facts for the factual-recall evaluation
(reference ``bergson/recall/facts.py:32-101``).

Name / town / employer / university lists are read from ``<data_dir>/names/*.txt`` and
paraphrase templates from ``<data_dir>/templates/*.txt`` when those files exist;
otherwise deterministic built-in lists are used (pronounceable names composed from
syllables, a fixed set of templates), so the benchmark runs without any data files.
"""

from __future__ import annotations

import itertools
import os
import random
from dataclasses import asdict, dataclass
from datetime import datetime, timedelta

FIELDS = ("birthplace", "birthdate", "employer", "university")

QUESTION_TEMPLATES = {
    "birthdate": "When was {first_name} {last_name} born?",
    "birthplace": "Where was {first_name} {last_name} born?",
    "employer": "Where does {first_name} {last_name} work?",
    "university": "What university did {first_name} {last_name} attend?",
}

BUILTIN_TEMPLATES = {
    "birthplace": ["{first_name} {last_name} was born in {birthplace}.",
                   "The birthplace of {first_name} {last_name} is {birthplace}.",
                   "{birthplace} is where {first_name} {last_name} was born."],
    "birthdate": ["{first_name} {last_name} was born on {birthdate}.",
                  "The date of birth of {first_name} {last_name} is {birthdate}.",
                  "On {birthdate}, {first_name} {last_name} was born."],
    "employer": ["{first_name} {last_name} works at {employer}.",
                 "{first_name} {last_name} is employed by {employer}.",
                 "The employer of {first_name} {last_name} is {employer}."],
    "university": ["{first_name} {last_name} studied at {university}.",
                   "{first_name} {last_name} is a graduate of {university}.",
                   "The university {first_name} {last_name} attended is {university}."],
}

_ONSETS = ["b", "br", "c", "d", "f", "g", "h", "j", "k", "l", "m", "n", "p", "r", "s", "st", "t", "v", "w", "z"]
_VOWELS = ["a", "e", "i", "o", "u", "ai", "ea", "ou"]
_CODAS = ["", "n", "r", "s", "l", "th", "m", "nd"]


def _syllable_words(count: int, syllables: int, salt: str) -> list[str]:
    """``count`` distinct capitalised words, in an order fixed by ``salt``."""
    parts = [o + v + c for o, v, c in itertools.product(_ONSETS, _VOWELS, _CODAS)]
    rng = random.Random(salt)
    seen, out = set(), []
    while len(out) < count:
        w = "".join(rng.choice(parts) for _ in range(syllables)).capitalize()
        if w not in seen:
            seen.add(w)
            out.append(w)
    return out


def _read_list(path: str) -> list[str] | None:
    if not os.path.isfile(path):
        return None
    with open(path) as f:
        return [line.strip() for line in f if line.strip()]


def load_name_lists(data_dir: str) -> dict[str, list[str]]:
    base = os.path.join(data_dir, "names")
    towns = _syllable_words(200, 2, "town")
    return {
        "first_name": _read_list(os.path.join(base, "first_name.txt")) or _syllable_words(10000, 2, "first"),
        "last_name": _read_list(os.path.join(base, "last_name.txt")) or _syllable_words(20000, 3, "last"),
        "employer": _read_list(os.path.join(base, "employer.txt")) or [f"{w} Systems" for w in _syllable_words(80, 2, "emp")],
        "town": _read_list(os.path.join(base, "town.txt")) or towns,
        "university": _read_list(os.path.join(base, "university.txt")) or [f"University of {w}" for w in towns[:100]],
    }


def load_templates(data_dir: str) -> dict[str, list[str]]:
    return {f: _read_list(os.path.join(data_dir, "templates", f"{f}.txt")) or BUILTIN_TEMPLATES[f] for f in FIELDS}


@dataclass(frozen=True)
class Profile:
    identifier: int
    first_name: str
    last_name: str
    birthdate: datetime
    birthplace: str
    employer: str
    university: str


def generate_profiles(seed: int = 0, path: str = "data"):
    rng = random.Random(seed)
    lists = load_name_lists(path)
    for key in ("first_name", "last_name", "employer", "town", "university"):
        rng.shuffle(lists[key])
    start, end = datetime(1995, 7, 2), datetime(2000, 2, 14)
    for i, (first, last) in enumerate(zip(lists["first_name"], lists["last_name"])):
        born = start + timedelta(days=rng.randint(0, (end - start).days))
        yield Profile(i, first, last, born, employer=rng.choice(lists["employer"]),
                      birthplace=rng.choice(lists["town"]), university=rng.choice(lists["university"]))


def fact_generator(num_facts: int, path: str = "data", seed: int = 0):
    """Rows ``{answer, fact, field, identifier, question, template}``: every paraphrase of
    every (person, field) fact until ``num_facts`` (person, field) pairs were emitted."""
    templates = load_templates(path)
    for profile in generate_profiles(seed, path):
        kw = asdict(profile)
        kw["birthdate"] = profile.birthdate.strftime("%d %B %Y")
        for field in FIELDS:
            for i, t in enumerate(templates[field]):
                yield {"answer": kw[field], "fact": t.format(**kw), "field": field, "identifier": profile.identifier,
                       "question": QUESTION_TEMPLATES[field].format(**kw), "template": i}
            num_facts -= 1
            if num_facts <= 0:
                return
