"""Build and cache the statements / questions datasets of the recall evaluation
(reference ``bergson/recall/generate.py``).  ``python -m bergson_b200.recall.generate
--num_people 1000`` generates them ahead of a run."""

from __future__ import annotations

from pathlib import Path

from datasets import Dataset

from ..config.config import RecallDataConfig
from .facts import fact_generator

NUM_FIELDS = 4


def recall_dataset_paths(cfg: RecallDataConfig) -> tuple[Path, Path]:
    tag = f"{cfg.num_people}p_seed{cfg.seed}" + ("_single" if cfg.single_paraphrase else "")
    d = Path(cfg.data_dir)
    return d / f"statements_{tag}.hf", d / f"questions_{tag}.hf"


def ensure_recall_datasets(cfg: RecallDataConfig) -> tuple[Path, Path]:
    s_path, q_path = recall_dataset_paths(cfg)
    if s_path.exists() and q_path.exists():
        print(f"Reusing cached recall datasets at {s_path} and {q_path}")
        return s_path, q_path
    statements, questions, seen = [], [], set()
    for row in fact_generator(NUM_FIELDS * cfg.num_people, cfg.data_dir, cfg.seed):
        if cfg.single_paraphrase and row["template"] != 0:
            continue
        statements.append(row)
        key = (row["identifier"], row["field"])
        if key not in seen:
            seen.add(key)
            questions.append({"question": row["question"], "answer": row["answer"],
                              "text": f"{row['question']} {row['answer']}", "field": row["field"],
                              "identifier": row["identifier"]})
    people = len({s["identifier"] for s in statements})
    if people < cfg.num_people:
        raise ValueError(f"Only generated {people} of the requested {cfg.num_people} people; the name lists in "
                         f"{cfg.data_dir}/names are too small.")
    s_path.parent.mkdir(parents=True, exist_ok=True)
    Dataset.from_list(statements).save_to_disk(str(s_path))
    Dataset.from_list(questions).save_to_disk(str(q_path))
    print(f"Generated {len(statements)} statements and {len(questions)} questions for {people} people")
    return s_path, q_path


if __name__ == "__main__":
    import sys

    from ..config.parsing import DataclassArgumentParser

    ensure_recall_datasets(DataclassArgumentParser(RecallDataConfig).parse(sys.argv[1:]))
