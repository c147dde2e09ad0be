"""B200-native decode attention (drop-in for the stream_attention decode path)."""
