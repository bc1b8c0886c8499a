"""On-disk formats of T5X checkpoints, written from the format descriptions: the Flax msgpack
index (`msgpack_io`) and zarr v2 arrays as TensorStore's zarr driver lays them out (`zarr_io`)."""
