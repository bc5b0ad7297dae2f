"""Table sizing exactly as the reference computes it (dlrm_s_pytorch.py:1236-1242, 309-322)."""
from __future__ import annotations


def hot_rows(total_categories: int, compress_rate: float, hash_rate: float, dim: int) -> int:
    """hotn: rows of the shared hot table = capacity `lim` of the sketch.  The factor 4D/(4D+48)
    charges each hot row its 48 bytes of sketch state.  Evaluated left to right in double, as in
    dlrm_s_pytorch.py:1239-1240."""
    return int(total_categories * compress_rate * (1 - hash_rate) * (dim * 4 / (dim * 4 + 48)))


def hash_rows(num_categories: int, compress_rate: float, hash_rate: float) -> int:
    """Rows of one field's hash table: round(cr*hr*n + 0.51), Python round-half-even
    (dlrm_s_pytorch.py:319 with hash_rate already multiplied by compress_rate at :1241)."""
    return round((compress_rate * hash_rate) * num_categories + 0.51)


def is_sketch_field(num_categories: int, compress_rate: float) -> bool:
    """Fields this small keep a plain full table (dlrm_s_pytorch.py:309)."""
    return num_categories > 2000 * compress_rate


def field_offsets(num_categories) -> list[int]:
    """f_offset: sum of the cardinalities of ALL earlier fields (dlrm_s_pytorch.py:351-353)."""
    out, tot = [], 0
    for n in num_categories:
        out.append(tot)
        tot += int(n)
    return out


def shard_hot_rows(num_categories, local_fields, compress_rate: float, hash_rate: float, dim: int, by: str = "fields") -> int:
    """Hot-table capacity of one shard of a field-sharded model.  The reference has one sketch and one hot table for
    all fields (dlrm_s_pytorch.py:1239-1240, 444-449); a shard owns a part of that capacity: in proportion to its
    number of fields ("fields": equal lookups per call meet equal capacity, whatever the fields' cardinalities) or
    what the reference's formula gives for the shard's own fields alone ("rows": a shard that holds only small fields
    then gets a sketch of a few buckets, or none).  Never below the 20 rows the sketch needs for a non-empty LRU
    stage (sketch.cpp:51-52)."""
    cards = [int(n) for n in num_categories]
    mine = list(local_fields)
    if by == "fields":
        return max(20, hot_rows(sum(cards), compress_rate, hash_rate, dim) * len(mine) // len(cards))
    if by == "rows":
        return max(20, hot_rows(sum(cards[f] for f in mine), compress_rate, hash_rate, dim))
    raise ValueError("hot_rows_by must be 'fields' or 'rows'")
