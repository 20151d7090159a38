"""Mirror of the reference's ``engine`` package for the hot path only."""
