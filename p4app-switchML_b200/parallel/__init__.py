"""Data-parallel plumbing: the Context binding, gradient bucketing over symmetric
memory, the DDP communication hook and the ``sml`` process group."""
