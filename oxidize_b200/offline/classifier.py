"""A small tabular classifier: CSV in, one-hidden-layer MLP trained with AdamW, accuracy out (the CSV half of the
reference's ``oxidize-train`` crate: ``load_csv_dataset`` ``src/lib.rs:521``, ``MlpClassifier`` ``:203``,
``train_classifier`` ``:447``; its video classifiers need ffmpeg and are not built).

    python -m oxidize_b200.offline.classifier --train-csv data.csv [--label-column N] [--epochs 20] [--save model.pt]

Rows are numeric features with the class label (an integer, or any string: labels are numbered in order of appearance) in
``label_column`` (default: the last column).  A header line is skipped when its fields are not numbers.  Features are
standardised with the training set's mean and deviation.
"""
from __future__ import annotations

import argparse
import csv
import sys
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch


@dataclass
class Dataset:
    inputs: np.ndarray  # [n, features] float32
    labels: np.ndarray  # [n] int64
    classes: List[str]


def load_csv_dataset(path: str, label_column: Optional[int] = None) -> Dataset:
    rows: List[List[str]] = []
    with open(path, newline="") as f:
        for rec in csv.reader(f):
            if rec and any(c.strip() for c in rec):
                rows.append([c.strip() for c in rec])
    if not rows:
        raise ValueError(f"{path}: empty")

    def numeric(v: str) -> bool:
        try:
            float(v)
            return True
        except ValueError:
            return False

    width = len(rows[0])
    col = width - 1 if label_column is None else label_column
    if not 0 <= col < width:
        raise ValueError(f"label column {col} outside the {width} columns")
    if not all(numeric(v) for i, v in enumerate(rows[0]) if i != col):
        rows = rows[1:]  # header
    names: Dict[str, int] = {}
    xs, ys = [], []
    for ln, rec in enumerate(rows, 1):
        if len(rec) != width:
            raise ValueError(f"{path}: row {ln} has {len(rec)} fields, expected {width}")
        try:
            xs.append([float(v) for i, v in enumerate(rec) if i != col])
        except ValueError:
            raise ValueError(f"{path}: row {ln} has a non-numeric feature") from None
        ys.append(names.setdefault(rec[col], len(names)))
    if len(names) < 2:
        raise ValueError(f"{path}: need at least two classes")
    return Dataset(np.asarray(xs, dtype=np.float32), np.asarray(ys, dtype=np.int64), list(names))


class MlpClassifier(torch.nn.Module):
    def __init__(self, input_size: int, hidden_size: int, classes: int, seed: int = 42):
        super().__init__()
        torch.manual_seed(seed)
        self.net = torch.nn.Sequential(torch.nn.Linear(input_size, hidden_size), torch.nn.ReLU(),
                                       torch.nn.Linear(hidden_size, classes))
        self.register_buffer("mean", torch.zeros(input_size))
        self.register_buffer("std", torch.ones(input_size))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.net((x - self.mean) / self.std)

    def predict(self, inputs: np.ndarray) -> np.ndarray:
        with torch.no_grad():
            return self(torch.from_numpy(np.asarray(inputs, dtype=np.float32))).argmax(dim=1).numpy()


def train_classifier(data: Dataset, epochs: int = 20, batch_size: int = 32, learning_rate: float = 1e-3, weight_decay: float = 0.01,
                     hidden_size: int = 128, seed: int = 42) -> Tuple[MlpClassifier, List[float]]:
    """Returns (model, mean loss per epoch)."""
    model = MlpClassifier(data.inputs.shape[1], hidden_size, len(data.classes), seed)
    x, y = torch.from_numpy(data.inputs), torch.from_numpy(data.labels)
    model.mean.copy_(x.mean(dim=0))
    model.std.copy_(x.std(dim=0).clamp_min(1e-6))
    opt = torch.optim.AdamW(model.net.parameters(), lr=learning_rate, weight_decay=weight_decay)
    gen = torch.Generator().manual_seed(seed)
    history = []
    for _ in range(epochs):
        order = torch.randperm(len(y), generator=gen)
        total = 0.0
        for i in range(0, len(y), batch_size):
            idx = order[i : i + batch_size]
            opt.zero_grad(set_to_none=True)
            loss = torch.nn.functional.cross_entropy(model(x[idx]), y[idx])
            loss.backward()
            opt.step()
            total += float(loss.detach()) * len(idx)
        history.append(total / len(y))
    return model, history


def evaluate_classifier(model: MlpClassifier, data: Dataset) -> Tuple[float, float]:
    """(accuracy, mean cross-entropy)."""
    with torch.no_grad():
        logits = model(torch.from_numpy(data.inputs))
        y = torch.from_numpy(data.labels)
        return float((logits.argmax(dim=1) == y).float().mean()), float(torch.nn.functional.cross_entropy(logits, y))


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="oxidize train-classifier", description="Train an MLP classifier on a CSV file")
    ap.add_argument("--train-csv", required=True)
    ap.add_argument("--eval-csv")
    ap.add_argument("--label-column", type=int, default=None)
    ap.add_argument("--epochs", type=int, default=20)
    ap.add_argument("--batch-size", type=int, default=32)
    ap.add_argument("--learning-rate", type=float, default=1e-3)
    ap.add_argument("--weight-decay", type=float, default=0.01)
    ap.add_argument("--hidden-size", type=int, default=128)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--save", help="write the trained model (torch state dict + class names) here")
    a = ap.parse_args(argv)
    try:
        data = load_csv_dataset(a.train_csv, a.label_column)
        model, hist = train_classifier(data, a.epochs, a.batch_size, a.learning_rate, a.weight_decay, a.hidden_size, a.seed)
        acc, loss = evaluate_classifier(model, data)
        print(f"train: {len(data.labels)} rows, {data.inputs.shape[1]} features, {len(data.classes)} classes; "
              f"loss {hist[0]:.4f} -> {hist[-1]:.4f}; accuracy {acc:.3f}")
        if a.eval_csv:
            ev = load_csv_dataset(a.eval_csv, a.label_column)
            remap = {c: i for i, c in enumerate(data.classes)}
            if any(c not in remap for c in ev.classes):
                raise ValueError("the evaluation file has classes the training file lacks")
            ev.labels = np.asarray([remap[ev.classes[i]] for i in ev.labels], dtype=np.int64)
            acc, loss = evaluate_classifier(model, ev)
            print(f"eval: {len(ev.labels)} rows; loss {loss:.4f}; accuracy {acc:.3f}")
        if a.save:
            torch.save({"state": model.state_dict(), "classes": data.classes, "hidden_size": a.hidden_size}, a.save)
    except (ValueError, OSError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    return 0


if __name__ == "__main__":
    sys.exit(main())
