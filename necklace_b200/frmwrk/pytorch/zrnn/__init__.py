"""ZeRO ("zr") helpers."""
from .zrfn import (bcast_to_zero_parallel_region, zr_pg_all_gather, zr_pg_all_reduce,
                   zr_pg_bcast, zr_pg_reduce, zr_pg_split)
