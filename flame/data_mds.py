from ttcd_b200.train.data_mds import MDSPretokenizedDataset, build_mds_dataset, parse_mds_uri  # noqa: F401
