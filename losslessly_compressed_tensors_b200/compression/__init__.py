"""Host-side construction of the exponent codebooks (probabilities -> Huffman tables)."""
