from ttcd_b200.train.data import *  # noqa: F401,F403
from ttcd_b200.train.data import (BufferShuffledIterableDataset, DataCollatorForLanguageModeling,  # noqa: F401
                                  OnlineTokenizedIterableDataset, ParallelAwareDataLoader, build_dataloader, build_dataset)
