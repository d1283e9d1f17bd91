"""Token data: synthetic Zipf streams and the pre-tokenised parquet shard reader."""
