"""Process plumbing: ranks, process groups, collectives over objects, cross-rank consensus,
filesystem scope, node load throttling and bounded device waits."""
