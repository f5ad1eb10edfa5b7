from .datasets import (InMemoryDataset, DataLoader, load_mnist_idx, load_cifar10_bin, synthetic_mnist,  # noqa: F401
                       synthetic_cifar10, gaussian_clusters, TokenShardDataset, write_token_shard, augment)
