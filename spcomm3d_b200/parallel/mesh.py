"""X x Y x Z process mesh and its torch.distributed sub-groups.

Rank order is z fastest, `rank = (x*Y + y)*Z + z`: the order of the MPI
Cartesian communicator every reference benchmark builds
(miniapp/bench_spmm.cpp:137-149).  The reference's serial helper class
src/Mesh3D.hpp:12-63 numbers ranks x fastest instead; `order="x_fastest"`
reproduces that for the simulators.  X splits sparse rows, Y splits sparse
columns, Z splits the dense inner dimension k (and replicates S).
"""
from __future__ import annotations

from dataclasses import dataclass, field


def dims_create(nranks: int, z: int = 1) -> tuple[int, int, int]:
    """Mesh shape for `nranks` with Z fixed: X*Y = nranks/Z split as evenly as
    possible with X >= Y (what MPI_Dims_create(size,3,{0,0,c}) returns,
    miniapp/bench_spmm.cpp:137-143).  8 ranks: z=2 -> 2x2x2, z=1 -> 4x2x1,
    z=8 -> 1x1x8."""
    if z <= 0 or nranks % z:
        raise ValueError(f"Z={z} does not divide {nranks} ranks")
    xy = nranks // z
    y = int(xy ** 0.5)
    while xy % y:
        y -= 1
    return xy // y, y, z


def split_k(k: int, Z: int, z: int) -> tuple[int, int]:
    """(offset, width) of z's slice of the inner dimension:
    width = k//Z + (z < k%Z) (miniapp/bench_spmm.cpp:167-172)."""
    base, rem = divmod(k, Z)
    return z * base + min(z, rem), base + (1 if z < rem else 0)


def split_nnz(nnz: int, Z: int, z: int) -> tuple[int, int]:
    """(offset, length) of the slice of a block's nonzero values that fiber
    rank z owns after the SDDMM reduction: nnz//Z (+1 for the first nnz%Z)
    (src/parallel_io.hpp:168-171, src/comm_setup.cpp:682-687)."""
    return split_k(nnz, Z, z)


@dataclass(frozen=True)
class Mesh3D:
    X: int
    Y: int
    Z: int
    order: str = "z_fastest"

    def __post_init__(self):
        if min(self.X, self.Y, self.Z) < 1:
            raise ValueError("mesh dims must be >= 1")
        if self.order not in ("z_fastest", "x_fastest"):
            raise ValueError("order must be z_fastest or x_fastest")

    @staticmethod
    def parse(text: str) -> "Mesh3D":
        x, y, z = (int(t) for t in text.lower().split("x"))
        return Mesh3D(x, y, z)

    @property
    def size(self) -> int:
        return self.X * self.Y * self.Z

    @property
    def xy_size(self) -> int:
        return self.X * self.Y

    def rank_of(self, x: int, y: int, z: int) -> int:
        if not (0 <= x < self.X and 0 <= y < self.Y and 0 <= z < self.Z):
            raise ValueError("coords outside mesh")
        if self.order == "z_fastest":
            return (x * self.Y + y) * self.Z + z
        return x + self.X * y + self.X * self.Y * z

    def coords_of(self, rank: int) -> tuple[int, int, int]:
        if not 0 <= rank < self.size:
            raise ValueError("rank outside mesh")
        if self.order == "z_fastest":
            return rank // (self.Y * self.Z), (rank // self.Z) % self.Y, rank % self.Z
        return rank % self.X, (rank // self.X) % self.Y, rank // (self.X * self.Y)

    def xy_rank(self, x: int, y: int) -> int:
        """Rank inside an xy plane (row-major in x, y)."""
        return x * self.Y + y

    def all_coords(self):
        return [self.coords_of(r) for r in range(self.size)]

    # fibers through a rank (src/Mesh3D.hpp:46-63)
    def neighbors_x(self, rank: int):
        _, y, z = self.coords_of(rank)
        return [self.rank_of(i, y, z) for i in range(self.X)]

    def neighbors_y(self, rank: int):
        x, _, z = self.coords_of(rank)
        return [self.rank_of(x, j, z) for j in range(self.Y)]

    def neighbors_z(self, rank: int):
        x, y, _ = self.coords_of(rank)
        return [self.rank_of(x, y, k) for k in range(self.Z)]

    def xy_plane(self, rank: int):
        _, _, z = self.coords_of(rank)
        return [self.rank_of(i, j, z) for i in range(self.X) for j in range(self.Y)]

    def __str__(self):
        return f"{self.X}x{self.Y}x{self.Z}"


@dataclass
class MeshGroups:
    """torch.distributed groups for one rank of a mesh.

    `row` = ranks sharing my (x, z), varying y: the peers A/Y rows move between;
    `col` = ranks sharing my (y, z), varying x: the peers B/X rows move between;
    `fiber` = ranks sharing my (x, y), varying z: the SDDMM value reduction;
    `plane` = my xy plane.  Group-local rank of a peer equals its varying
    coordinate (y, x, z and x*Y+y respectively).
    """
    mesh: Mesh3D
    rank: int
    world: object = None
    row: object = None
    col: object = None
    fiber: object = None
    plane: object = None
    coords: tuple = field(default=(0, 0, 0))

    @staticmethod
    def create(mesh: Mesh3D, rank: int | None = None) -> "MeshGroups":
        import torch.distributed as dist
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        if dist.get_world_size() != mesh.size:
            raise ValueError(f"mesh {mesh} needs {mesh.size} ranks, world has {dist.get_world_size()}")
        rank = dist.get_rank() if rank is None else rank
        g = MeshGroups(mesh, rank, world=dist.group.WORLD, coords=mesh.coords_of(rank))
        x0, y0, z0 = g.coords
        # every rank must create every group, in the same order
        for x in range(mesh.X):
            for z in range(mesh.Z):
                grp = dist.new_group([mesh.rank_of(x, y, z) for y in range(mesh.Y)])
                if (x, z) == (x0, z0):
                    g.row = grp
        for y in range(mesh.Y):
            for z in range(mesh.Z):
                grp = dist.new_group([mesh.rank_of(x, y, z) for x in range(mesh.X)])
                if (y, z) == (y0, z0):
                    g.col = grp
        for x in range(mesh.X):
            for y in range(mesh.Y):
                grp = dist.new_group([mesh.rank_of(x, y, z) for z in range(mesh.Z)])
                if (x, y) == (x0, y0):
                    g.fiber = grp
        for z in range(mesh.Z):
            grp = dist.new_group([mesh.rank_of(x, y, z) for x in range(mesh.X) for y in range(mesh.Y)])
            if z == z0:
                g.plane = grp
        return g
