"""Integration layer: attention dispatch and Ulysses context parallelism for the sparse path."""
