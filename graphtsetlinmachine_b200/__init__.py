"""B200-native engine for the Graph Tsetlin Machine fit / predict path behind the reference's Python API."""
