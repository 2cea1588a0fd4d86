"""Vision input and tower: image decode / resize / patch rows (`processor`), the tower's configuration,
host metadata and CPU restatement (`tower`), and the device tower (`tower_gpu`)."""
