"""MovieLens ``ratings.csv`` (+ optional ``movies.csv`` join) as an iterable of row dicts (``torchrec/datasets/movielens.py``)."""
from __future__ import annotations

import csv
import os
from typing import Any, Callable, Dict, Iterator, List, Optional, Union

from torch.utils.data import IterableDataset

RATINGS_FILENAME = "ratings.csv"
MOVIES_FILENAME = "movies.csv"
DEFAULT_RATINGS_COLUMN_NAMES: List[str] = ["userId", "movieId", "rating", "timestamp"]
DEFAULT_MOVIES_COLUMN_NAMES: List[str] = ["movieId", "title", "genres"]
DEFAULT_COLUMN_NAMES: List[str] = DEFAULT_RATINGS_COLUMN_NAMES + DEFAULT_MOVIES_COLUMN_NAMES[1:]
COLUMN_TYPE_CASTERS: List[Callable[[str], Union[float, int, str]]] = [lambda v: safe_cast(v, int, 0), lambda v: safe_cast(v, int, 0), lambda v: safe_cast(v, float, 0.0),
                                                                       lambda v: safe_cast(v, int, 0), lambda v: safe_cast(v, str, ""), lambda v: safe_cast(v, str, "")]


def safe_cast(val: Any, dest_type: Callable[[Any], Any], default: Any) -> Any:
    try:
        return dest_type(val)
    except (ValueError, TypeError):
        return default


def _default_row_mapper(example: List[str]) -> Dict[str, Union[float, int, str]]:
    return {DEFAULT_COLUMN_NAMES[idx]: COLUMN_TYPE_CASTERS[idx](val) for idx, val in enumerate(example)}


class _MovieLens(IterableDataset):
    def __init__(self, root: str, include_movies_data: bool, row_mapper: Optional[Callable[[List[str]], Any]], **open_kw: Any) -> None:
        self.root, self.include_movies_data, self.row_mapper, self.open_kw = root, include_movies_data, row_mapper, open_kw

    def __iter__(self) -> Iterator[Any]:
        movies: Dict[str, List[str]] = {}
        if self.include_movies_data:
            with open(os.path.join(self.root, MOVIES_FILENAME), newline="", **self.open_kw) as f:
                r = csv.reader(f)
                next(r, None)
                for row in r:
                    movies[row[0]] = row[1:]
        with open(os.path.join(self.root, RATINGS_FILENAME), newline="", **self.open_kw) as f:
            r = csv.reader(f)
            next(r, None)
            for row in r:
                if self.include_movies_data:
                    row = row + movies.get(row[1], ["", ""])
                yield self.row_mapper(row) if self.row_mapper else row


def movielens_20m(root: str, *, include_movies_data: bool = False, row_mapper=_default_row_mapper, **open_kw: Any) -> IterableDataset:
    return _MovieLens(root, include_movies_data, row_mapper, **open_kw)


def movielens_25m(root: str, *, include_movies_data: bool = False, row_mapper=_default_row_mapper, **open_kw: Any) -> IterableDataset:
    return _MovieLens(root, include_movies_data, row_mapper, **open_kw)
