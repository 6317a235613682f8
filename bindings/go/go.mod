module github.com/spiraltorch-b200/bindings/go

go 1.21
