"""Geometry helpers shared by camera-conditioned models: camera / quaternion math and volume rendering."""
